// Dense reconstruction  int4/int2 -> fp16/fp32 [K, N]  (the reference's vecquant*recons_*).
//
// HBM-bound: per weight 0.5 B are read and 2 B (fp16) written.  One thread owns one packed
// word-row r and 8 adjacent columns: it reads its 8 words with two 128-bit loads (each word
// exactly once device-wide), and writes 8 output rows as one 128-bit store each, so a warp
// writes 512 contiguous bytes per row.  Scales and zero points are fetched per output row
// from g_idx[k] (act-order safe) but only re-read when the group changes.
#include "q4_common.cuh"

namespace q4 {

// ---- 4-bit, v2 ------------------------------------------------------------------------------
// fp16: w = rn(rn(s*q) - rn(s*(z+1))): the three roundings of the reference's c10::Half
// arithmetic (quant_cuda_kernel.cu:1142-1151); mul.rn / sub.rn forbid contraction into an FMA.
struct GroupRowH {
  __half2 s[4];    // scales of the 8 columns
  __half2 zp[4];   // rn(s * (z+1))
};

__device__ __forceinline__ void load_group_h(GroupRowH& gr, const __half* scales, const uint32_t* qzeros,
                                             int g, int N, int n0) {
  uint4 sv = *reinterpret_cast<const uint4*>(scales + (size_t)g * N + n0);
  uint32_t zw = qzeros[(size_t)g * (N >> 3) + (n0 >> 3)];
  gr.s[0] = as_h2(sv.x); gr.s[1] = as_h2(sv.y); gr.s[2] = as_h2(sv.z); gr.s[3] = as_h2(sv.w);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t za = ((zw >> (8 * c)) & 0xF) + 1, zb = ((zw >> (8 * c + 4)) & 0xF) + 1;   // 1..16
    __half2 z1 = __halves2half2(__ushort2half_rn((unsigned short)za), __ushort2half_rn((unsigned short)zb));
    gr.zp[c] = __hmul2_rn(gr.s[c], z1);
  }
}

template <int BYTE, bool ODD>
__device__ __forceinline__ void recons_row_h(__half* out_row, const uint32_t (&w)[8], const GroupRowH& gr) {
  uint4 o;
  uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    __half2 q = nibble_pair<BYTE, ODD>(w[2 * c], w[2 * c + 1]);
    ov[c] = as_u32(__hsub2_rn(__hmul2_rn(gr.s[c], q), gr.zp[c]));
  }
  *reinterpret_cast<uint4*>(out_row) = o;
}

__global__ void __launch_bounds__(256)
recons4_v2_h_kernel(const uint32_t* __restrict__ qw, __half* __restrict__ out, const __half* __restrict__ scales,
                    const uint32_t* __restrict__ qzeros, const int* __restrict__ g_idx, int R, int N) {
  const int oct = blockIdx.x * blockDim.x + threadIdx.x;    // column octet
  const int r = blockIdx.y * blockDim.y + threadIdx.y;      // packed row
  if (oct >= (N >> 3) || r >= R) return;
  const int n0 = oct << 3;
  const uint32_t* src = qw + (size_t)r * N + n0;
  uint4 a = ldg_stream(src), b = ldg_stream(src + 4);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  const int4 ga = *reinterpret_cast<const int4*>(g_idx + 8 * r);
  const int4 gb = *reinterpret_cast<const int4*>(g_idx + 8 * r + 4);
  const int g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
  __half* dst = out + (size_t)(8 * r) * N + n0;
  GroupRowH gr;
  int cur = -1;
#define Q4_ROW(J, BYTE, ODD)                                                     \
  if (g[J] != cur) { cur = g[J]; load_group_h(gr, scales, qzeros, cur, N, n0); } \
  recons_row_h<BYTE, ODD>(dst + (size_t)(J) * N, w, gr);
  Q4_ROW(0, 0, false) Q4_ROW(1, 0, true) Q4_ROW(2, 1, false) Q4_ROW(3, 1, true)
  Q4_ROW(4, 2, false) Q4_ROW(5, 2, true) Q4_ROW(6, 3, false) Q4_ROW(7, 3, true)
#undef Q4_ROW
}

// fp32 scales: zero = rn32(s*(z+1)); w = fma(s, q, -zero) — what nvcc emits for the reference's
// `scale * q - zero` on floats (default -fmad=true).
__global__ void __launch_bounds__(256)
recons4_v2_f_kernel(const uint32_t* __restrict__ qw, float* __restrict__ out, const float* __restrict__ scales,
                    const uint32_t* __restrict__ qzeros, const int* __restrict__ g_idx, int R, int N) {
  const int oct = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y * blockDim.y + threadIdx.y;
  if (oct >= (N >> 3) || r >= R) return;
  const int n0 = oct << 3;
  const uint32_t* src = qw + (size_t)r * N + n0;
  uint4 a = ldg_stream(src), b = ldg_stream(src + 4);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float s[8], zero[8];
  int cur = -1;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int g = g_idx[8 * r + j];
    if (g != cur) {
      cur = g;
      const float4 s0 = *reinterpret_cast<const float4*>(scales + (size_t)g * N + n0);
      const float4 s1 = *reinterpret_cast<const float4*>(scales + (size_t)g * N + n0 + 4);
      s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
      const uint32_t zw = qzeros[(size_t)g * (N >> 3) + (n0 >> 3)];
#pragma unroll
      for (int c = 0; c < 8; ++c) zero[c] = __fmul_rn(s[c], (float)(((zw >> (4 * c)) & 0xF) + 1));
    }
    float o[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) o[c] = __fmaf_rn(s[c], (float)((w[c] >> (4 * j)) & 0xF), -zero[c]);
    float4* d = reinterpret_cast<float4*>(out + (size_t)(8 * r + j) * N + n0);
    d[0] = make_float4(o[0], o[1], o[2], o[3]);
    d[1] = make_float4(o[4], o[5], o[6], o[7]);
  }
}

// ---- 4-bit, v1: W = scales[n]*q - zeros[n] (quant_cuda_kernel.cu:1085-1096) ------------------------
template <typename T>
__global__ void __launch_bounds__(256)
recons4_v1_kernel(const uint32_t* __restrict__ qw, T* __restrict__ out, const T* __restrict__ scales,
                  const T* __restrict__ zeros, int R, int N) {
  const int oct = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y * blockDim.y + threadIdx.y;
  if (oct >= (N >> 3) || r >= R) return;
  const int n0 = oct << 3;
  const uint32_t* src = qw + (size_t)r * N + n0;
  uint4 a = ldg_stream(src), b = ldg_stream(src + 4);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  T s[8], z[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) { s[c] = scales[n0 + c]; z[c] = zeros[n0 + c]; }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    T* d = out + (size_t)(8 * r + j) * N + n0;
    if constexpr (sizeof(T) == 2) {
      uint4 o;
      __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        oh[c] = __hsub_rn(__hmul_rn(s[c], __ushort2half_rn((unsigned short)((w[c] >> (4 * j)) & 0xF))), z[c]);
      *reinterpret_cast<uint4*>(d) = o;
    } else {
      float o[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) o[c] = __fmaf_rn(s[c], (float)((w[c] >> (4 * j)) & 0xF), -z[c]);
      reinterpret_cast<float4*>(d)[0] = make_float4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<float4*>(d)[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
  }
}

// ---- 2-bit, v2 (quant_cuda_kernel.cu:1185-1211): 16 rows per word, zero field + 1 ---------------
template <typename T>
__global__ void __launch_bounds__(256)
recons2_v2_kernel(const uint32_t* __restrict__ qw, T* __restrict__ out, const T* __restrict__ scales,
                  const uint32_t* __restrict__ qzeros, const int* __restrict__ g_idx, int R, int N) {
  const int oct = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y * blockDim.y + threadIdx.y;
  if (oct >= (N >> 3) || r >= R) return;
  const int n0 = oct << 3;
  const uint32_t* src = qw + (size_t)r * N + n0;
  uint4 a = ldg_stream(src), b = ldg_stream(src + 4);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  T s[8], zero[8];
  int cur = -1;
  for (int j = 0; j < 16; ++j) {
    const int g = g_idx[16 * r + j];
    if (g != cur) {
      cur = g;
      const uint32_t zw = qzeros[(size_t)g * (N >> 4) + (n0 >> 4)];
      const int zoff = (n0 & 15) * 2;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        s[c] = scales[(size_t)g * N + n0 + c];
        const unsigned z1 = ((zw >> (zoff + 2 * c)) & 0x3) + 1;
        if constexpr (sizeof(T) == 2) zero[c] = __hmul_rn(s[c], __ushort2half_rn((unsigned short)z1));
        else zero[c] = __fmul_rn(s[c], (float)z1);
      }
    }
    T* d = out + (size_t)(16 * r + j) * N + n0;
    if constexpr (sizeof(T) == 2) {
      uint4 o;
      __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        oh[c] = __hsub_rn(__hmul_rn(s[c], __ushort2half_rn((unsigned short)((w[c] >> (2 * j)) & 0x3))), zero[c]);
      *reinterpret_cast<uint4*>(d) = o;
    } else {
      float o[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) o[c] = __fmaf_rn(s[c], (float)((w[c] >> (2 * j)) & 0x3), -zero[c]);
      reinterpret_cast<float4*>(d)[0] = make_float4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<float4*>(d)[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
  }
}

static int recons_args_ok(const void* qweight, const void* out, const void* scales, const void* z,
                          int K, int N, int per, int dtype) {
  if (!qweight || !out || !scales || !z) return fail(Q4_E_BADARG, "recons: null pointer");
  if (K <= 0 || N <= 0) return fail(Q4_E_BADARG, "recons: K=%d N=%d must be positive", K, N);
  if (dtype != Q4_F16 && dtype != Q4_F32) return fail(Q4_E_BADARG, "recons: unknown dtype %d", dtype);
  if (K % per || N % per || N % 8) return fail(Q4_E_SHAPE, "recons: K=%d N=%d must be multiples of %d", K, N, per);
  if (!aligned16(qweight) || !aligned16(out) || !aligned16(scales))
    return fail(Q4_E_ALIGN, "recons: qweight/out/scales must be 16-byte aligned");
  return check_device();
}

static void recons_grid(int R, int N, dim3& grid, dim3& block) {
  const int octs = N >> 3;
  const int bx = octs >= 64 ? 64 : 32;
  block = dim3(bx, 256 / bx);
  grid = dim3((octs + bx - 1) / bx, (R + block.y - 1) / block.y);
}

}  // namespace q4

using namespace q4;

extern "C" int q4_recons_v2(const int32_t* qweight, void* out, const void* scales, const int32_t* qzeros,
                            const int32_t* g_idx, int K, int N, int G, int dtype, q4_stream_t stream) {
  if (int e = recons_args_ok(qweight, out, scales, qzeros, K, N, 8, dtype)) return e;
  if (!g_idx) return fail(Q4_E_BADARG, "recons_v2: g_idx is null");
  if (G <= 0) return fail(Q4_E_BADARG, "recons_v2: G=%d", G);
  if (!aligned16(g_idx)) return fail(Q4_E_ALIGN, "recons_v2: g_idx must be 16-byte aligned");
  dim3 grid, block;
  recons_grid(K / 8, N, grid, block);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q4_F16)
    recons4_v2_h_kernel<<<grid, block, 0, st>>>((const uint32_t*)qweight, (__half*)out, (const __half*)scales,
                                                (const uint32_t*)qzeros, g_idx, K / 8, N);
  else
    recons4_v2_f_kernel<<<grid, block, 0, st>>>((const uint32_t*)qweight, (float*)out, (const float*)scales,
                                                (const uint32_t*)qzeros, g_idx, K / 8, N);
  return check_cuda(cudaGetLastError(), "recons_v2 launch");
}

extern "C" int q4_recons_v1(const int32_t* qweight, void* out, const void* scales, const void* zeros,
                            int K, int N, int dtype, q4_stream_t stream) {
  if (int e = recons_args_ok(qweight, out, scales, zeros, K, N, 8, dtype)) return e;
  dim3 grid, block;
  recons_grid(K / 8, N, grid, block);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q4_F16)
    recons4_v1_kernel<__half><<<grid, block, 0, st>>>((const uint32_t*)qweight, (__half*)out,
                                                      (const __half*)scales, (const __half*)zeros, K / 8, N);
  else
    recons4_v1_kernel<float><<<grid, block, 0, st>>>((const uint32_t*)qweight, (float*)out,
                                                     (const float*)scales, (const float*)zeros, K / 8, N);
  return check_cuda(cudaGetLastError(), "recons_v1 launch");
}

extern "C" int q2_recons_v2(const int32_t* qweight, void* out, const void* scales, const int32_t* qzeros,
                            const int32_t* g_idx, int K, int N, int G, int dtype, q4_stream_t stream) {
  if (int e = recons_args_ok(qweight, out, scales, qzeros, K, N, 16, dtype)) return e;
  if (!g_idx) return fail(Q4_E_BADARG, "recons2_v2: g_idx is null");
  if (G <= 0) return fail(Q4_E_BADARG, "recons2_v2: G=%d", G);
  dim3 grid, block;
  recons_grid(K / 16, N, grid, block);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q4_F16)
    recons2_v2_kernel<__half><<<grid, block, 0, st>>>((const uint32_t*)qweight, (__half*)out, (const __half*)scales,
                                                      (const uint32_t*)qzeros, g_idx, K / 16, N);
  else
    recons2_v2_kernel<float><<<grid, block, 0, st>>>((const uint32_t*)qweight, (float*)out, (const float*)scales,
                                                     (const uint32_t*)qzeros, g_idx, K / 16, N);
  return check_cuda(cudaGetLastError(), "recons2_v2 launch");
}
