// The element-wise work of a LLaMA decoder layer around the quantised linears, one kernel each way instead
// of the half-dozen framework kernels the stock modules launch: RMSNorm, the SwiGLU product and the rotary
// embedding, forward and backward.  All of it is bound by HBM (every operand crosses once), fp16 in and out,
// fp32 arithmetic inside.  The norm weights and the rotary tables are frozen in a LoRA finetune (only the
// LoRA factors train), so the backward kernels produce input gradients only.
#include "q4_common.cuh"

namespace q4 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// block-wide sum, result on every thread; `red` holds one float per warp
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ---- RMSNorm: y = w * half(x * rsqrt(mean(x^2) + eps)), the two roundings of LlamaRMSNorm.forward -------
// One CTA per row; a thread keeps its 8-element vectors of the row in registers between the two passes.
constexpr int RN_THREADS = 256, RN_VEC = 4;             // rows of up to 256 * 4 * 8 = 8192 elements

__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_fwd_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ y, float* __restrict__ rstd,
                   int H, float eps) {
  __shared__ float red[RN_THREADS / 32];
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const int nv = H >> 3;
  uint4 v[RN_VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int j = threadIdx.x + i * RN_THREADS;
    v[i] = j < nv ? xr[j] : make_uint4(0u, 0u, 0u, 0u);
    const float2 a = __half22float2(as_h2(v[i].x)), b = __half22float2(as_h2(v[i].y));
    const float2 c = __half22float2(as_h2(v[i].z)), d = __half22float2(as_h2(v[i].w));
    ss += (a.x * a.x + a.y * a.y) + (b.x * b.x + b.y * b.y) + (c.x * c.x + c.y * c.y) + (d.x * d.x + d.y * d.y);
  }
  const float r = rsqrtf(block_sum(ss, red) / (float)H + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int j = threadIdx.x + i * RN_THREADS;
    if (j >= nv) continue;
    const uint4 wv = wr[j];
    auto one = [&](uint32_t xv, uint32_t ww) {
      const float2 f = __half22float2(as_h2(xv));
      return as_u32(__hmul2(as_h2(ww), __floats2half2_rn(f.x * r, f.y * r)));
    };
    yr[j] = make_uint4(one(v[i].x, wv.x), one(v[i].y, wv.y), one(v[i].z, wv.z), one(v[i].w, wv.w));
  }
}

// dx = rstd * (g - xh * mean(g * xh)),  g = dy * w,  xh = x * rstd
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_bwd_kernel(const __half* __restrict__ dy, const __half* __restrict__ x, const __half* __restrict__ w,
                   const float* __restrict__ rstd, __half* __restrict__ dx, int H) {
  __shared__ float red[RN_THREADS / 32];
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* gr = reinterpret_cast<const uint4*>(dy + row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const int nv = H >> 3;
  const float r = rstd[row];
  float g[RN_VEC][8], xh[RN_VEC][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int j = threadIdx.x + i * RN_THREADS;
    const bool ok = j < nv;
    const uint4 xv = ok ? xr[j] : make_uint4(0u, 0u, 0u, 0u), gv = ok ? gr[j] : make_uint4(0u, 0u, 0u, 0u);
    const uint4 wv = ok ? wr[j] : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, gs[4] = {gv.x, gv.y, gv.z, gv.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 xf = __half22float2(as_h2(xs[q])), gf = __half22float2(as_h2(gs[q])), wf = __half22float2(as_h2(ws[q]));
      xh[i][2 * q] = xf.x * r; xh[i][2 * q + 1] = xf.y * r;
      g[i][2 * q] = gf.x * wf.x; g[i][2 * q + 1] = gf.y * wf.y;
      dot += g[i][2 * q] * xh[i][2 * q] + g[i][2 * q + 1] * xh[i][2 * q + 1];
    }
  }
  const float m = block_sum(dot, red) / (float)H;
  uint4* dr = reinterpret_cast<uint4*>(dx + row * H);
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int j = threadIdx.x + i * RN_THREADS;
    if (j >= nv) continue;
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
      o[q] = as_u32(__floats2half2_rn(r * (g[i][2 * q] - xh[i][2 * q] * m), r * (g[i][2 * q + 1] - xh[i][2 * q + 1] * m)));
    dr[j] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- SwiGLU: out = half(silu(gate)) * up ------------------------------------------------------------------
// gate and up are rows of pitch `pitch` halves (two tensors, or the two halves of one fused gate_up output).

__global__ void swiglu_fwd_kernel(const __half* __restrict__ gate, const __half* __restrict__ up, __half* __restrict__ out,
                                  int rows, int I, int pitch) {
  const int nv = I >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (size_t)rows * nv; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / nv, j = idx - r * nv;
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + r * pitch + 8 * j), uv = *reinterpret_cast<const uint4*>(up + r * pitch + 8 * j);
    auto one = [&](uint32_t gg, uint32_t uu) {
      const float2 f = __half22float2(as_h2(gg));
      return as_u32(__hmul2(__floats2half2_rn(silu_f(f.x), silu_f(f.y)), as_h2(uu)));
    };
    *reinterpret_cast<uint4*>(out + r * I + 8 * j) = make_uint4(one(gv.x, uv.x), one(gv.y, uv.y), one(gv.z, uv.z), one(gv.w, uv.w));
  }
}

// d_gate = d_out * up * silu'(gate),  d_up = d_out * silu(gate);  silu'(v) = s (1 + v (1 - s)),  s = sigmoid(v)
__global__ void swiglu_bwd_kernel(const __half* __restrict__ dout, const __half* __restrict__ gate, const __half* __restrict__ up,
                                  __half* __restrict__ dgate, __half* __restrict__ dup, int rows, int I, int pitch, int dpitch) {
  const int nv = I >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (size_t)rows * nv; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / nv, j = idx - r * nv;
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + r * pitch + 8 * j), uv = *reinterpret_cast<const uint4*>(up + r * pitch + 8 * j);
    const uint4 dv = *reinterpret_cast<const uint4*>(dout + r * I + 8 * j);
    const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w}, us[4] = {uv.x, uv.y, uv.z, uv.w}, ds[4] = {dv.x, dv.y, dv.z, dv.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 gf = __half22float2(as_h2(gs[q])), uf = __half22float2(as_h2(us[q])), df = __half22float2(as_h2(ds[q]));
      const float s0 = 1.f / (1.f + __expf(-gf.x)), s1 = 1.f / (1.f + __expf(-gf.y));
      og[q] = as_u32(__floats2half2_rn(df.x * uf.x * s0 * (1.f + gf.x * (1.f - s0)), df.y * uf.y * s1 * (1.f + gf.y * (1.f - s1))));
      ou[q] = as_u32(__floats2half2_rn(df.x * gf.x * s0, df.y * gf.y * s1));
    }
    *reinterpret_cast<uint4*>(dgate + r * dpitch + 8 * j) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dup + r * dpitch + 8 * j) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// ---- rotary embedding on [tokens, heads, D] (the memory order of a projection's output) -----------------
// out[d] = t[d] cos[d] + rot[d] sin[d],  rot[d] = -t[d + D/2] for d < D/2, t[d - D/2] otherwise; cos / sin [tokens, D].
// Backward (the transpose): dt[d] = g[d] cos[d] + (d < D/2 ? g[d + D/2] sin[d + D/2] : -g[d - D/2] sin[d - D/2]).
// A thread handles 8 elements of the low half together with their 8 partners of the high half.
template <bool BWD>
__global__ void rope_kernel(const __half* __restrict__ in, const __half* __restrict__ cos, const __half* __restrict__ sin,
                            __half* __restrict__ out, int tokens, int heads, int D, int in_pitch, int table_rows) {
  const int half_v = D >> 4;                             // 8-element vectors per half head
  const size_t total = (size_t)tokens * heads * half_v;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t th = idx / half_v;
    const int j = (int)(idx - th * half_v);
    const size_t tok = th / heads;
    const int h = (int)(th - tok * heads);
    const __half* src = in + tok * in_pitch + (size_t)h * D;
    const uint4 lo = *reinterpret_cast<const uint4*>(src + 8 * j), hi = *reinterpret_cast<const uint4*>(src + (D >> 1) + 8 * j);
    const size_t trow = tok % (size_t)table_rows;           // tables of one sequence serve every sequence of the batch
    const __half* cr = cos + trow * D;
    const __half* sr = sin + trow * D;
    const uint4 cl = *reinterpret_cast<const uint4*>(cr + 8 * j), ch = *reinterpret_cast<const uint4*>(cr + (D >> 1) + 8 * j);
    const uint4 sl = *reinterpret_cast<const uint4*>(sr + 8 * j), sh = *reinterpret_cast<const uint4*>(sr + (D >> 1) + 8 * j);
    const uint32_t L[4] = {lo.x, lo.y, lo.z, lo.w}, Hh[4] = {hi.x, hi.y, hi.z, hi.w};
    const uint32_t CL[4] = {cl.x, cl.y, cl.z, cl.w}, CH[4] = {ch.x, ch.y, ch.z, ch.w};
    const uint32_t SL[4] = {sl.x, sl.y, sl.z, sl.w}, SH[4] = {sh.x, sh.y, sh.z, sh.w};
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = __half22float2(as_h2(L[q])), b = __half22float2(as_h2(Hh[q]));
      const float2 c0 = __half22float2(as_h2(CL[q])), c1 = __half22float2(as_h2(CH[q]));
      const float2 s0 = __half22float2(as_h2(SL[q])), s1 = __half22float2(as_h2(SH[q]));
      if (!BWD) {
        ol[q] = as_u32(__floats2half2_rn(a.x * c0.x - b.x * s0.x, a.y * c0.y - b.y * s0.y));
        oh[q] = as_u32(__floats2half2_rn(b.x * c1.x + a.x * s1.x, b.y * c1.y + a.y * s1.y));
      } else {
        ol[q] = as_u32(__floats2half2_rn(a.x * c0.x + b.x * s1.x, a.y * c0.y + b.y * s1.y));
        oh[q] = as_u32(__floats2half2_rn(b.x * c1.x - a.x * s0.x, b.y * c1.y - a.y * s0.y));
      }
    }
    __half* dst = out + (tok * heads + h) * (size_t)D;
    *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
    *reinterpret_cast<uint4*>(dst + (D >> 1) + 8 * j) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
}

static int ew_grid(size_t work_items, int threads) {
  const size_t want = (work_items + threads - 1) / threads;
  const size_t cap = (size_t)sm_count() * 16;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace q4

using namespace q4;

extern "C" int q4_rmsnorm_fwd(const void* x, const void* weight, void* y, float* rstd, int rows, int H, float eps, q4_stream_t stream) {
  if (!x || !weight || !y) return fail(Q4_E_BADARG, "rmsnorm: null pointer");
  if (rows <= 0 || H <= 0) return fail(Q4_E_BADARG, "rmsnorm: rows=%d H=%d", rows, H);
  if (H % 8 || H > RN_THREADS * RN_VEC * 8) return fail(Q4_E_SHAPE, "rmsnorm: H=%d must be a multiple of 8, at most %d", H, RN_THREADS * RN_VEC * 8);
  if (!aligned16(x) || !aligned16(weight) || !aligned16(y)) return fail(Q4_E_ALIGN, "rmsnorm: pointers must be 16-byte aligned");
  if (int e = check_device()) return e;
  rmsnorm_fwd_kernel<<<rows, RN_THREADS, 0, (cudaStream_t)stream>>>((const __half*)x, (const __half*)weight, (__half*)y, rstd, H, eps);
  return check_cuda(cudaGetLastError(), "rmsnorm launch");
}

extern "C" int q4_rmsnorm_bwd(const void* dy, const void* x, const void* weight, const float* rstd, void* dx, int rows, int H,
                              q4_stream_t stream) {
  if (!dy || !x || !weight || !rstd || !dx) return fail(Q4_E_BADARG, "rmsnorm_bwd: null pointer");
  if (rows <= 0 || H <= 0) return fail(Q4_E_BADARG, "rmsnorm_bwd: rows=%d H=%d", rows, H);
  if (H % 8 || H > RN_THREADS * RN_VEC * 8) return fail(Q4_E_SHAPE, "rmsnorm_bwd: H=%d must be a multiple of 8, at most %d", H, RN_THREADS * RN_VEC * 8);
  if (!aligned16(dy) || !aligned16(x) || !aligned16(weight) || !aligned16(dx)) return fail(Q4_E_ALIGN, "rmsnorm_bwd: pointers must be 16-byte aligned");
  if (int e = check_device()) return e;
  rmsnorm_bwd_kernel<<<rows, RN_THREADS, 0, (cudaStream_t)stream>>>((const __half*)dy, (const __half*)x, (const __half*)weight, rstd, (__half*)dx, H);
  return check_cuda(cudaGetLastError(), "rmsnorm_bwd launch");
}

extern "C" int q4_swiglu_fwd(const void* gate, const void* up, void* out, int rows, int I, int pitch, q4_stream_t stream) {
  if (!gate || !up || !out) return fail(Q4_E_BADARG, "swiglu: null pointer");
  if (rows <= 0 || I <= 0 || pitch < I) return fail(Q4_E_BADARG, "swiglu: rows=%d I=%d pitch=%d", rows, I, pitch);
  if (I % 8 || pitch % 8) return fail(Q4_E_SHAPE, "swiglu: I=%d and pitch=%d must be multiples of 8", I, pitch);
  if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return fail(Q4_E_ALIGN, "swiglu: pointers must be 16-byte aligned");
  if (int e = check_device()) return e;
  swiglu_fwd_kernel<<<ew_grid((size_t)rows * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>((const __half*)gate, (const __half*)up, (__half*)out, rows, I, pitch);
  return check_cuda(cudaGetLastError(), "swiglu launch");
}

extern "C" int q4_swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, int rows, int I, int pitch,
                             int dpitch, q4_stream_t stream) {
  if (!dout || !gate || !up || !dgate || !dup) return fail(Q4_E_BADARG, "swiglu_bwd: null pointer");
  if (rows <= 0 || I <= 0 || pitch < I || dpitch < I) return fail(Q4_E_BADARG, "swiglu_bwd: rows=%d I=%d pitch=%d dpitch=%d", rows, I, pitch, dpitch);
  if (I % 8 || pitch % 8 || dpitch % 8) return fail(Q4_E_SHAPE, "swiglu_bwd: sizes must be multiples of 8");
  if (!aligned16(dout) || !aligned16(gate) || !aligned16(up) || !aligned16(dgate) || !aligned16(dup))
    return fail(Q4_E_ALIGN, "swiglu_bwd: pointers must be 16-byte aligned");
  if (int e = check_device()) return e;
  swiglu_bwd_kernel<<<ew_grid((size_t)rows * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __half*)dout, (const __half*)gate, (const __half*)up, (__half*)dgate, (__half*)dup, rows, I, pitch, dpitch);
  return check_cuda(cudaGetLastError(), "swiglu_bwd launch");
}

extern "C" int q4_rope(const void* in, const void* cos, const void* sin, void* out, int tokens, int heads, int D, int in_pitch,
                       int table_rows, int backward, q4_stream_t stream) {
  if (!in || !cos || !sin || !out) return fail(Q4_E_BADARG, "rope: null pointer");
  if (table_rows <= 0 || tokens % table_rows) return fail(Q4_E_BADARG, "rope: %d tokens are not a whole number of tables of %d rows", tokens, table_rows);
  if (tokens <= 0 || heads <= 0 || D <= 0 || in_pitch < heads * D) return fail(Q4_E_BADARG, "rope: tokens=%d heads=%d D=%d pitch=%d", tokens, heads, D, in_pitch);
  if (D % 16 || in_pitch % 8) return fail(Q4_E_SHAPE, "rope: D=%d must be a multiple of 16 and the pitch of 8", D);
  if (!aligned16(in) || !aligned16(cos) || !aligned16(sin) || !aligned16(out)) return fail(Q4_E_ALIGN, "rope: pointers must be 16-byte aligned");
  if (int e = check_device()) return e;
  const int grid = ew_grid((size_t)tokens * heads * (D / 16), 256);
  if (backward) rope_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half*)in, (const __half*)cos, (const __half*)sin, (__half*)out, tokens, heads, D, in_pitch, table_rows);
  else rope_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half*)in, (const __half*)cos, (const __half*)sin, (__half*)out, tokens, heads, D, in_pitch, table_rows);
  return check_cuda(cudaGetLastError(), "rope launch");
}
