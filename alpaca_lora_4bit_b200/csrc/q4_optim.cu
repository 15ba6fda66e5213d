// The optimiser of a LoRA finetune over ONE flat fp32 buffer: every trainable factor is a view of `param`,
// every gradient a view of `grad` (the buffer the data-parallel ranks all-reduce), so a step is three launches
// whatever the number of adapters: a scan for non-finite gradients, AdamW with the unscaling folded in, and
// the loss-scale bookkeeping.  The reference leaves this to the HF Trainer (finetune.py:150-170:
// optim="adamw_torch", fp16=True, i.e. AdamW under fp16 autocast with a dynamic loss scale, a step with
// non-finite gradients being skipped); the arithmetic here is torch.optim.AdamW's (decoupled weight decay,
// bias-corrected moments) and torch.amp.GradScaler's.
//
// All state that changes from step to step lives on the device, so that the step can sit inside a CUDA graph:
//   state[0] steps taken, state[1] loss scale, state[2] steps since the scale last changed, state[3] 1 if the
//   scan found a non-finite gradient in this step (all fp32).
#include "q4_common.cuh"

namespace q4 {

constexpr int OPT_THREADS = 256;

__global__ void __launch_bounds__(OPT_THREADS)
flat_nonfinite_kernel(const float* __restrict__ grad, size_t n, float* __restrict__ state) {
  bool bad = false;
  const size_t n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(grad);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = __ldg(g4 + i);
    // finite values have an exponent field below all-ones
    bad |= ((__float_as_uint(v.x) & 0x7F800000u) == 0x7F800000u) | ((__float_as_uint(v.y) & 0x7F800000u) == 0x7F800000u) |
           ((__float_as_uint(v.z) & 0x7F800000u) == 0x7F800000u) | ((__float_as_uint(v.w) & 0x7F800000u) == 0x7F800000u);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) bad |= (__float_as_uint(grad[(n4 << 2) + threadIdx.x]) & 0x7F800000u) == 0x7F800000u;
  if (__syncthreads_or(bad) && threadIdx.x == 0) state[3] = 1.f;     // every writer writes the same value
}

__global__ void __launch_bounds__(OPT_THREADS)
flat_adamw_kernel(float* __restrict__ param, const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, size_t n,
                  float lr, float beta1, float beta2, float eps, float weight_decay, float grad_div, const float* __restrict__ state,
                  __half* __restrict__ shadow) {
  if (state[3] != 0.f) return;                                       // non-finite gradients: the step is skipped
  const float step = state[0] + 1.f;
  const float inv = 1.f / (state[1] * grad_div);
  const float bc1 = 1.f - powf(beta1, step), bc2 = 1.f - powf(beta2, step);
  const float step_size = lr / bc1, inv_sqrt_bc2 = rsqrtf(bc2), decay = 1.f - lr * weight_decay;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float g = grad[i] * inv;
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float pn = param[i] * decay - step_size * (mi / (sqrtf(vi) * inv_sqrt_bc2 + eps));
    param[i] = pn;
    if (shadow) shadow[i] = __float2half_rn(pn);                       // the fp16 copy the kernels of the next step read
  }
}

__global__ void scale_update_kernel(float* state, float growth, float backoff, int interval) {
  if (state[3] != 0.f) {
    if (interval > 0) state[1] *= backoff;
    state[2] = 0.f;
    state[3] = 0.f;
  } else {
    state[0] += 1.f;
    const float since = state[2] + 1.f;
    if (interval > 0 && since >= (float)interval) {
      state[1] *= growth;
      state[2] = 0.f;
    } else {
      state[2] = since;
    }
  }
}

}  // namespace q4

using namespace q4;

extern "C" int q4_adamw_flat(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, size_t n, float lr, float beta1,
                             float beta2, float eps, float weight_decay, float grad_div, float* state, float growth, float backoff,
                             int growth_interval, void* half_shadow, q4_stream_t stream) {
  if (!param || !grad || !exp_avg || !exp_avg_sq || !state) return fail(Q4_E_BADARG, "adamw_flat: null pointer");
  if (n == 0) return Q4_OK;
  if (!aligned16(grad)) return fail(Q4_E_ALIGN, "adamw_flat: the gradient buffer must be 16-byte aligned");
  if (!(grad_div > 0.f) || !(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f))
    return fail(Q4_E_BADARG, "adamw_flat: grad_div=%g beta1=%g beta2=%g", (double)grad_div, (double)beta1, (double)beta2);
  if (int e = check_device()) return e;
  const cudaStream_t st = (cudaStream_t)stream;
  const size_t want = (n + OPT_THREADS - 1) / OPT_THREADS;
  const int grid = (int)(want < (size_t)(8 * sm_count()) ? want : (size_t)(8 * sm_count()));
  flat_nonfinite_kernel<<<grid, OPT_THREADS, 0, st>>>(grad, n, state);
  flat_adamw_kernel<<<grid, OPT_THREADS, 0, st>>>(param, grad, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, grad_div, state,
                                                  (__half*)half_shadow);
  scale_update_kernel<<<1, 1, 0, st>>>(state, growth, backoff, growth_interval);
  return check_cuda(cudaGetLastError(), "adamw_flat launch");
}
