// Decode product  y[M,N] (+)= x[M,K] * W  for 1 <= M <= 16 straight from the packed int4 layer.
//
// Bound by HBM: per weight 0.5 B of qweight plus 1/64 B of scales and 1/256 B of zero points at
// groupsize 128; x and y are noise.  Design:
//   * A CTA owns 32 adjacent columns and one K-split; its 8 warps walk the split in chunks of
//     128 rows (4 "steps" of 32 rows).  In a step lane (g,t) reads ONE 128-bit word group:
//     packed row 4*step+t, columns 4g..4g+3, so a warp covers 4 packed rows x 128 contiguous
//     bytes and every byte of qweight is requested once, with four such loads in flight per lane.
//   * Nibbles are turned into fp16 with the exponent trick (w & 0x000F000F | 0x6400 = 1024+q,
//     one LOP3 per two weights) and fed to mma.sync.m16n8k16 as the A operand (rows = 16 output
//     columns); x is the B operand (columns = batch).  The contraction index of the MMA is
//     free, so the (q_j, q_j+4) pairing that the mask produces is matched by permuting x with
//     four PRMTs per step instead of un-shuffling the weights.
//   * The +1024 offset and the zero point leave with one extra MMA against an all-ones A tile,
//     which yields sum_k x[k] per batch column:  y += s * (acc - (1024 + z + 1) * xsum), applied
//     once per quantisation group in fp32.
//   * Cross-warp reduction in shared memory, cross-split reduction through a caller-provided
//     workspace with a per-tile arrival counter: the last CTA to arrive adds the partials in
//     split order, so the result does not depend on scheduling.  No atomics on y, no zero-fill.
// The act-order variant (group from g_idx per row) cannot factor the scale out of the
// contraction; it dequantises per element from shared-memory scale tables instead.
#include "q4_common.cuh"

namespace q4 {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_TN = 32;          // columns per CTA
// Workspace layout: a fixed 64 KiB head of arrival counters (one per column tile, so the
// counters of one shape never alias the partial sums of another), then the partial sums.
constexpr size_t GEMV_WS_HEAD = 65536;

struct GemvParams {
  const __half* x;
  const uint32_t* qw;
  void* y;
  const __half* scales;
  const uint32_t* qzeros;
  const int* g_idx;
  const __half* bias;
  float* part;                        // [S][M][N] partial sums (only S > 1)
  unsigned* counters;                 // [N/32] arrival counters, zero between launches
  int M, K, N, groupsize;
  int steps_total, steps_per_split, S;
  int y_f32, accumulate;
  int v1;                             // v1 layer: scales fp16 [N], qzeros reinterpreted as fp16 zeros [N]
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void store_y(const GemvParams& p, int b, int n, float v) {
  if (p.bias) v += __half2float(p.bias[n]);
  const size_t o = (size_t)b * p.N + n;
  if (p.y_f32) {
    float* y = reinterpret_cast<float*>(p.y);
    y[o] = p.accumulate ? y[o] + v : v;
  } else {
    __half* y = reinterpret_cast<__half*>(p.y);
    y[o] = __float2half_rn(p.accumulate ? __half2float(y[o]) + v : v);
  }
}

// Cross-warp (shared memory) and cross-split (workspace) reduction; `red` is [8][MT*8][32].
template <int MT>
__device__ __forceinline__ void gemv_reduce_store(const GemvParams& p, float* red, const float (&yacc)[MT][2][4],
                                                  int c0, int split) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  __shared__ int s_last;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = 4 * g + 2 * j + (i >> 1), b = mt * 8 + 2 * t + (i & 1);
        red[(warp * (MT * 8) + b) * GEMV_TN + col] = yacc[mt][j][i];
      }
  __syncthreads();
  const int col = threadIdx.x & 31;
  float v[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int b = mt * 8 + (threadIdx.x >> 5);
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) s += red[(w * (MT * 8) + b) * GEMV_TN + col];
    v[mt] = s;
  }
  if (p.S == 1) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int b = mt * 8 + (threadIdx.x >> 5);
      if (b < p.M) store_y(p, b, c0 + col, v[mt]);
    }
    return;
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int b = mt * 8 + (threadIdx.x >> 5);
    if (b < p.M) __stcg(p.part + ((size_t)split * p.M + b) * p.N + c0 + col, v[mt]);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counters + blockIdx.x, 1u) == (unsigned)(p.S - 1));
  __syncthreads();
  if (!s_last) return;
  __threadfence();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int b = mt * 8 + (threadIdx.x >> 5);
    if (b < p.M) {
      float s = 0.f;
      for (int sp = 0; sp < p.S; ++sp) s += __ldcg(p.part + ((size_t)sp * p.M + b) * p.N + c0 + col);
      store_y(p, b, c0 + col, s);
    }
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0u;    // ready for the next launch
}

// ---- sequential groups (group of row k = k / groupsize) ------------------------------------------
template <int MT>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_seq_kernel(const GemvParams p) {
  __shared__ float red[GEMV_WARPS * MT * 8 * GEMV_TN];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c0 = blockIdx.x * GEMV_TN;
  const int split = blockIdx.y;
  const int sb = split * p.steps_per_split;
  const int se = min(sb + p.steps_per_split, p.steps_total);
  const int N = p.N, K = p.K;
  const int steps_per_group = p.groupsize >> 5;

  float yacc[MT][2][4];
  float c[MT][2][4], co[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) { yacc[mt][j][i] = 0.f; c[mt][j][i] = 0.f; }
#pragma unroll
    for (int i = 0; i < 4; ++i) co[mt][i] = 0.f;
  }

  const uint32_t* wp = p.qw + (size_t)t * N + c0 + 4 * g;          // + 4*step*N
  const __half* xp0 = p.x + (size_t)g * K + 8 * t;                  // + 32*step
  const bool xok0 = g < p.M, xok1 = (g + 8) < p.M;

  int cur_grp = -1;
  uint2 sc = make_uint2(0, 0), zh = make_uint2(0, 0);
  uint32_t zw = 0;

  auto flush = [&]() {
    // columns 4g..4g+3: scales as 4 halves, zero points as nibbles 4(g&1).. of the qzeros word
    const __half2 s01 = as_h2(sc.x), s23 = as_h2(sc.y);
    const float s[4] = {__low2float(s01), __high2float(s01), __low2float(s23), __high2float(s23)};
    float zz[4], zf[4];
    if (!p.v1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { zz[i] = 1025.f + (float)((zw >> (16 * (g & 1) + 4 * i)) & 0xF); zf[i] = 0.f; }
    } else {          // W = s*q - zero: only the 1024 offset scales with s, the float zero does not
      const __half2 z01 = as_h2(zh.x), z23 = as_h2(zh.y);
      zf[0] = __low2float(z01); zf[1] = __high2float(z01); zf[2] = __low2float(z23); zf[3] = __high2float(z23);
#pragma unroll
      for (int i = 0; i < 4; ++i) zz[i] = 1024.f;
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = 2 * j + (i >> 1);
          float v = fmaf(s[col], fmaf(-zz[col], co[mt][i & 1], c[mt][j][i]), yacc[mt][j][i]);
          yacc[mt][j][i] = fmaf(-zf[col], co[mt][i & 1], v);
          c[mt][j][i] = 0.f;
        }
#pragma unroll
      for (int i = 0; i < 4; ++i) co[mt][i] = 0.f;
    }
  };

  for (int s0 = sb + 4 * warp; s0 < se; s0 += 4 * GEMV_WARPS) {
    uint4 wv[4], xv[MT][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int step = s0 + i;
      if (step < se) {
        wv[i] = ldg_stream(wp + (size_t)(4 * step) * N);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const bool ok = mt ? xok1 : xok0;
          xv[mt][i] = ok ? __ldg(reinterpret_cast<const uint4*>(xp0 + (size_t)(8 * mt) * K + 32 * step))
                         : make_uint4(0, 0, 0, 0);
        }
      } else {
        wv[i] = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) xv[mt][i] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int step = s0 + i;
      if (step >= se) break;
      const int grp = step / steps_per_group;
      if (grp != cur_grp) {
        if (cur_grp >= 0) flush();
        cur_grp = grp;
        sc = __ldg(reinterpret_cast<const uint2*>(p.scales + (size_t)grp * N + c0 + 4 * g));
        if (!p.v1) zw = __ldg(p.qzeros + (size_t)grp * (N >> 3) + ((c0 + 4 * g) >> 3));
        else zh = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p.qzeros) + c0 + 4 * g));
      }
      const uint32_t w[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w};
      uint32_t pr[4][4];                      // pr[word][m] = (q_m, q_m+4) + 1024
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        pr[q][0] = (w[q] & 0x000F000Fu) | 0x64006400u;
        pr[q][1] = ((w[q] >> 4) & 0x000F000Fu) | 0x64006400u;
        pr[q][2] = ((w[q] >> 8) & 0x000F000Fu) | 0x64006400u;
        pr[q][3] = ((w[q] >> 12) & 0x000F000Fu) | 0x64006400u;
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint4 xq = xv[mt][i];             // x[k..k+7] of batch row g (+8)
        const uint32_t xb[4] = {prmt(xq.x, xq.z, 0x5410), prmt(xq.x, xq.z, 0x7632),    // (x0,x4) (x1,x5)
                                prmt(xq.y, xq.w, 0x5410), prmt(xq.y, xq.w, 0x7632)};   // (x2,x6) (x3,x7)
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          const uint32_t b0 = xb[2 * ks], b1 = xb[2 * ks + 1];
          mma16816(c[mt][0], pr[0][2 * ks], pr[1][2 * ks], pr[0][2 * ks + 1], pr[1][2 * ks + 1], b0, b1);
          mma16816(c[mt][1], pr[2][2 * ks], pr[3][2 * ks], pr[2][2 * ks + 1], pr[3][2 * ks + 1], b0, b1);
          mma16816(co[mt], 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, b0, b1);
        }
      }
    }
  }
  if (cur_grp >= 0) flush();
  gemv_reduce_store<MT>(p, red, yacc, c0, split);
}

// ---- act-order (group of row k = g_idx[k]) -------------------------------------------------------
// Scale and (z+1) of the CTA's 32 columns for every group live in shared memory as half2
// (s, z+1); every element is dequantised as s*(q - (z+1)) in fp16 pairs before the MMA.
template <int MT>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_act_kernel(const GemvParams p, int G) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* red = reinterpret_cast<float*>(smem_raw);                              // [8][MT*8][32]
  __half2* tab = reinterpret_cast<__half2*>(smem_raw + sizeof(float) * GEMV_WARPS * MT * 8 * GEMV_TN);  // [G][32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c0 = blockIdx.x * GEMV_TN;
  const int split = blockIdx.y;
  const int sb = split * p.steps_per_split;
  const int se = min(sb + p.steps_per_split, p.steps_total);
  const int N = p.N, K = p.K;

  for (int i = threadIdx.x; i < G * GEMV_TN; i += GEMV_THREADS) {
    const int grp = i >> 5, col = i & 31;
    const uint32_t zw = p.qzeros[(size_t)grp * (N >> 3) + ((c0 + col) >> 3)];
    const unsigned z1 = ((zw >> (4 * (col & 7))) & 0xF) + 1;
    tab[i] = __halves2half2(p.scales[(size_t)grp * N + c0 + col], __ushort2half_rn((unsigned short)z1));
  }
  __syncthreads();

  float yacc[MT][2][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) yacc[mt][j][i] = 0.f;

  const uint32_t* wp = p.qw + (size_t)t * N + c0 + 4 * g;
  const __half* xp0 = p.x + (size_t)g * K + 8 * t;
  const bool xok0 = g < p.M, xok1 = (g + 8) < p.M;

  for (int step = sb + warp; step < se; step += GEMV_WARPS) {
    const uint4 wv = ldg_stream(wp + (size_t)(4 * step) * N);
    const int k0 = 32 * step + 8 * t;
    const int4 ga = __ldg(reinterpret_cast<const int4*>(p.g_idx + k0));
    const int4 gb = __ldg(reinterpret_cast<const int4*>(p.g_idx + k0 + 4));
    const int gi[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
    const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t pr[4][4];                        // pr[word][m] = (w_m, w_m+4) dequantised
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const uint32_t raw = ((w[q] >> (4 * m)) & 0x000F000Fu) | 0x64006400u;
        const __half2 qq = __hsub2(as_h2(raw), as_h2(0x64006400u));              // (q_m, q_m+4)
        const __half2 ta = tab[gi[m] * GEMV_TN + 4 * g + q], tb = tab[gi[m + 4] * GEMV_TN + 4 * g + q];
        const __half2 sv = __lows2half2(ta, tb), zv = __highs2half2(ta, tb);
        pr[q][m] = as_u32(__hmul2(sv, __hsub2(qq, zv)));
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const bool ok = mt ? xok1 : xok0;
      const uint4 xq = ok ? __ldg(reinterpret_cast<const uint4*>(xp0 + (size_t)(8 * mt) * K + 32 * step))
                          : make_uint4(0, 0, 0, 0);
      const uint32_t xb[4] = {prmt(xq.x, xq.z, 0x5410), prmt(xq.x, xq.z, 0x7632),
                              prmt(xq.y, xq.w, 0x5410), prmt(xq.y, xq.w, 0x7632)};
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const uint32_t b0 = xb[2 * ks], b1 = xb[2 * ks + 1];
        mma16816(yacc[mt][0], pr[0][2 * ks], pr[1][2 * ks], pr[0][2 * ks + 1], pr[1][2 * ks + 1], b0, b1);
        mma16816(yacc[mt][1], pr[2][2 * ks], pr[3][2 * ks], pr[2][2 * ks + 1], pr[3][2 * ks + 1], b0, b1);
      }
    }
  }
  gemv_reduce_store<MT>(p, red, yacc, c0, split);
}

static void gemv_plan(int K, int N, int& S, int& steps_per_split) {
  const int tiles = N / GEMV_TN, steps = K / 32;
  int want = (592 + tiles - 1) / tiles;                 // about four CTAs per SM
  int cap = steps / 32; if (cap < 1) cap = 1;           // keep >= 1024 rows per split
  S = want < cap ? want : cap;
  if (S < 1) S = 1;
  steps_per_split = (steps + S - 1) / S;
  steps_per_split = (steps_per_split + 3) / 4 * 4;
  S = (steps + steps_per_split - 1) / steps_per_split;
}

}  // namespace q4

using namespace q4;

extern "C" size_t q4_gemv_workspace_bytes(int M, int K, int N) {
  if (M <= 0 || K <= 0 || N <= 0 || K % 32 || N % 32) return 0;
  int S, sps;
  gemv_plan(K, N, S, sps);
  return GEMV_WS_HEAD + (S > 1 ? (size_t)S * M * N * sizeof(float) : 0);
}

extern "C" int q4_gemv(const void* x, const int32_t* qweight, void* y, const void* scales,
                       const int32_t* qzeros, const int32_t* g_idx, const void* bias,
                       int M, int K, int N, int G, int groupsize, int y_dtype, unsigned flags,
                       void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  if (!x || !qweight || !y || !scales || !qzeros) return fail(Q4_E_BADARG, "gemv: null pointer");
  if (M < 1 || M > 16) return fail(Q4_E_SHAPE, "gemv: M=%d outside 1..16", M);
  if (K <= 0 || N <= 0 || G <= 0 || groupsize <= 0) return fail(Q4_E_BADARG, "gemv: K=%d N=%d G=%d groupsize=%d", K, N, G, groupsize);
  if (K % 32 || N % 32) return fail(Q4_E_SHAPE, "gemv: K=%d and N=%d must be multiples of 32", K, N);
  if (y_dtype != Q4_F16 && y_dtype != Q4_F32) return fail(Q4_E_BADARG, "gemv: unknown y_dtype %d", y_dtype);
  const bool act = flags & Q4_GEMV_ACT_ORDER;
  const bool v1 = flags & Q4_GEMV_V1;
  if (v1) {
    if (act) return fail(Q4_E_BADARG, "gemv: v1 layers have no g_idx");
    groupsize = K; G = 1;
  }
  if (act && !g_idx) return fail(Q4_E_BADARG, "gemv: act-order needs g_idx");
  if (!act && (groupsize % 32 || (size_t)G * groupsize < (size_t)K))
    return fail(Q4_E_SHAPE, "gemv: groupsize=%d must be a multiple of 32 and G*groupsize >= K", groupsize);
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(scales) || (act && !aligned16(g_idx)))
    return fail(Q4_E_ALIGN, "gemv: x/qweight/scales/g_idx must be 16-byte aligned");
  if ((K * 2) % 16) return fail(Q4_E_ALIGN, "gemv: row pitch of x must be a multiple of 16 bytes");
  if (int e = check_device()) return e;

  GemvParams p;
  p.x = (const __half*)x; p.qw = (const uint32_t*)qweight; p.y = y; p.scales = (const __half*)scales;
  p.qzeros = (const uint32_t*)qzeros; p.g_idx = g_idx; p.bias = (const __half*)bias;
  p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
  p.steps_total = K / 32;
  gemv_plan(K, N, p.S, p.steps_per_split);
  p.y_f32 = (y_dtype == Q4_F32); p.accumulate = (flags & Q4_GEMV_ACCUMULATE) ? 1 : 0; p.v1 = v1 ? 1 : 0;
  const size_t need = q4_gemv_workspace_bytes(M, K, N);
  if (p.S > 1) {
    if (!workspace || workspace_bytes < need)
      return fail(Q4_E_WORKSPACE, "gemv: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    if (!aligned16(workspace)) return fail(Q4_E_ALIGN, "gemv: workspace must be 16-byte aligned");
    if ((size_t)(N / GEMV_TN) * sizeof(unsigned) > GEMV_WS_HEAD)
      return fail(Q4_E_SHAPE, "gemv: N=%d has more column tiles than the workspace head holds", N);
    p.counters = (unsigned*)workspace;
    p.part = (float*)((char*)workspace + GEMV_WS_HEAD);
  } else {
    p.counters = nullptr; p.part = nullptr;
  }
  const dim3 grid(N / GEMV_TN, p.S), block(GEMV_THREADS);
  cudaStream_t st = (cudaStream_t)stream;
  if (!act) {
    if (M <= 8) gemv_seq_kernel<1><<<grid, block, 0, st>>>(p);
    else gemv_seq_kernel<2><<<grid, block, 0, st>>>(p);
  } else {
    const int MT = M <= 8 ? 1 : 2;
    const size_t smem = sizeof(float) * GEMV_WARPS * MT * 8 * GEMV_TN + (size_t)G * GEMV_TN * sizeof(__half2);
    if (smem > 200 * 1024) return fail(Q4_E_SHAPE, "gemv: act-order tables for G=%d groups do not fit shared memory", G);
    if (MT == 1) {
      if (int e = check_cuda(cudaFuncSetAttribute(gemv_act_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "gemv smem attr")) return e;
      gemv_act_kernel<1><<<grid, block, smem, st>>>(p, G);
    } else {
      if (int e = check_cuda(cudaFuncSetAttribute(gemv_act_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "gemv smem attr")) return e;
      gemv_act_kernel<2><<<grid, block, smem, st>>>(p, G);
    }
  }
  return check_cuda(cudaGetLastError(), "gemv launch");
}
