// The rank-r products of a LoRA adapter on a quantised layer that do not fit inside the dequant-GEMM kernels:
//   u  = (alpha / r) x A^T          [M, r]   before the forward GEMM (which adds u B^T to x W)
//   v  = (alpha / r) dy B           [M, r]   before the backward GEMM (which adds v A to dy W^T)
//   dA = v^T x   [r, K],  dB = dy^T u   [N, r]   the gradients of the two factors
// (Linear4bitLt.forward, models.py:58-66 of the reference, runs them as nn.Linear calls and leaves the gradients
// to autograd: four library GEMMs, two scalings and the padding copies per layer and pass.)  All four read one
// [M, wide] activation once and produce something tiny, so they are bound by that read; u and v leave in the
// [M, 64] zero-padded fp16 form the GEMM kernels take as their extra pipeline stage, and the gradients leave in
// fp32, the dtype of the factors.
#include "q4_async.cuh"
#include <atomic>

namespace q4 {

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t cluster_nctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ float ld_dsmem_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// ---- out [M, 64] = scale * X [M, C] W^T, W [r, C]; columns r..63 are written as zeros --------------------
// A CTA owns eight rows of X and walks the contraction in chunks (2048 elements for r <= 16) that arrive in shared
// memory as bulk copies, one per staged row (the eight rows of X and the r rows of W) on the chunk's mbarrier; its
// eight warps share a chunk (warp w takes the 32-element blocks w, w + 8, ...) and meet in shared memory at the end.
// What the forms of this kernel measured at 1024 rows x 4096: plain loads, 8.6 us (the compiler keeps one block's
// loads in flight per warp however the loop is written, so a row is walked in sixteen round trips to L2); the
// contraction split over a cluster of CTAs, 7.5-8.9 us (more warps, but a cluster launch alone costs 3 us);
// 16-byte cp.async copies of everything at once, 5.2 us (one SM pulls its 128 KB through the load/store path at
// 40-60 GB/s); bulk copies, 3.6 us (the two library kernels and the pad it replaces: 9.3 us + 3).
// A lane takes 16 contiguous bytes of its row of X and of its row of W per block: which four of the MMA's
// sixteen k-slots those eight elements occupy is the same for both operands, so the order of the sum is the
// only thing the re-mapping changes.  Rows 8..15 of the MMA tile stay zero.
constexpr int LP_ROWS = 8, LP_WARPS = 8, LP_THREADS = LP_WARPS * 32;
// chunk length and ring depth per output width: as much of the contraction in flight at once as shared memory holds
// (a CTA's time is the number of round trips to L2 it has to wait for, one after the other)
__host__ __device__ constexpr int lp_chunk(int nt) { return nt <= 2 ? 2048 : (nt == 4 ? 1024 : 512); }
__host__ __device__ constexpr int lp_stages(int nt) { return nt == 1 ? 3 : 2; }
__host__ __device__ constexpr int lp_pitch(int nt) { return lp_chunk(nt) * 2 + 16; }   // bytes per staged row; + 16 keeps the eight rows a quarter-warp reads on different banks

template <int NT>                                // 8-column tiles of the output that r reaches into
__global__ void __launch_bounds__(LP_THREADS)
lora_project_kernel(const __half* __restrict__ X, const __half* __restrict__ W, __half* __restrict__ out, int M, int C, int r, float scale) {
  extern __shared__ __align__(128) unsigned char lp_smem[];
  constexpr int ROWS = LP_ROWS + 8 * NT;         // staged rows per chunk: 8 of X, then 8 NT of W
  constexpr int LP_CHUNK = lp_chunk(NT), LP_PITCH = lp_pitch(NT), STAGE = ROWS * LP_PITCH, LP_NS = lp_stages(NT);
  float* red = reinterpret_cast<float*>(lp_smem + LP_NS * STAGE);          // [warps][8 rows][8 NT + 1]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int n_chunks = (C + LP_CHUNK - 1) / LP_CHUNK;

  // Rows past M and rows of W past r are staged from a valid row instead and dropped when the result is stored.
  // One bulk copy per staged row and chunk, issued by the thread of that row; the chunk's barrier counts the bytes.
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + LP_WARPS * LP_ROWS * (8 * NT + 1) + 1);
  bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(bars) + 7) & ~(uintptr_t)7);
  __shared__ int gave_up;
  if (threadIdx.x == 0) {
    for (int i = 0; i < LP_NS; ++i) mbar_init(&bars[i], 1);
    gave_up = 0;
    mbar_fence_init();
  }
  __syncthreads();
  auto load_chunk = [&](int c) {
    unsigned char* st = lp_smem + (c % LP_NS) * STAGE;
    const int k0 = c * LP_CHUNK, kn = min(LP_CHUNK, C - k0);               // elements of this chunk (a multiple of 32)
    if (threadIdx.x == 0) mbar_arrive_expect_tx(&bars[c % LP_NS], (uint32_t)(ROWS * kn * 2));
    __syncthreads();                             // the expectation is posted before any copy can complete on the barrier
    if (threadIdx.x < ROWS) {
      const int row = threadIdx.x;
      const __half* src = row < LP_ROWS ? X + (size_t)min(blockIdx.x * LP_ROWS + row, M - 1) * C
                                        : W + (size_t)min(row - LP_ROWS, r - 1) * C;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(st + row * LP_PITCH)), "l"(src + k0), "r"((uint32_t)(kn * 2)), "r"(smem_u32(&bars[c % LP_NS])) : "memory");
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
#pragma unroll
  for (int c = 0; c < LP_NS - 1; ++c)
    if (c < n_chunks) load_chunk(c);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + LP_NS - 1 < n_chunks) {
      __syncthreads();                           // everyone is done with chunk c - 1, whose slot the next copy overwrites
      load_chunk(c + LP_NS - 1);
    }
    {                                            // chunk c has landed (bounded wait: on expiry the result is dropped)
      const uint32_t parity = (uint32_t)((c / LP_NS) & 1);
      bool ok = mbar_test_wait(&bars[c % LP_NS], parity);
      for (uint32_t i = 0; !ok && i < (gave_up ? 4u : 4000000u); ++i) ok = mbar_test_wait(&bars[c % LP_NS], parity);
      if (!ok) gave_up = 1;
    }
    const unsigned char* st = lp_smem + (c % LP_NS) * STAGE;
    const int blocks = min(LP_CHUNK, C - c * LP_CHUNK) >> 5;
    for (int b = warp; b < blocks; b += LP_WARPS) {
      const uint4 xv = *reinterpret_cast<const uint4*>(st + g * LP_PITCH + 64 * b + 16 * t);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 wv = *reinterpret_cast<const uint4*>(st + (LP_ROWS + 8 * nt + g) * LP_PITCH + 64 * b + 16 * t);
        mma_f16_16816(acc[nt], xv.x, 0u, xv.y, 0u, wv.x, wv.y);
        mma_f16_16816(acc[nt], xv.z, 0u, xv.w, 0u, wv.z, wv.w);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    red[(warp * LP_ROWS + g) * (8 * NT + 1) + 8 * nt + 2 * t] = acc[nt][0];
    red[(warp * LP_ROWS + g) * (8 * NT + 1) + 8 * nt + 2 * t + 1] = acc[nt][1];
  }
  __syncthreads();
  // 8 rows x 32 column pairs: one half2 per thread
  const int orow = threadIdx.x >> 5, cp = threadIdx.x & 31;
  if (blockIdx.x * LP_ROWS + orow < M) {
    float s0 = 0.f, s1 = 0.f;
    if (2 * cp < 8 * NT) {
#pragma unroll
      for (int w = 0; w < LP_WARPS; ++w) {
        s0 += red[(w * LP_ROWS + orow) * (8 * NT + 1) + 2 * cp];
        s1 += red[(w * LP_ROWS + orow) * (8 * NT + 1) + 2 * cp + 1];
      }
    }
    if (2 * cp >= r) s0 = 0.f;
    if (2 * cp + 1 >= r) s1 = 0.f;
    reinterpret_cast<__half2*>(out + (size_t)(blockIdx.x * LP_ROWS + orow) * 64)[cp] = __floats2half2_rn(s0 * scale, s1 * scale);
  }
}

template <int NT> static size_t lora_project_smem() {
  return (size_t)lp_stages(NT) * (LP_ROWS + 8 * NT) * lp_pitch(NT) + (size_t)LP_WARPS * LP_ROWS * (8 * NT + 1) * sizeof(float) + 64;
}

// ---- out [j, c] (or out [c, j]) = sum over m of S [m, j] X [m, c], j < r, S of pitch 64 --------------------
// A small-by-tall-by-wide product bound by the one read of X.  A CTA owns 128 columns of X and a slice of the
// rows; 32-row stages of X and S arrive in shared memory through a three-deep cp.async ring (24 KB in flight per
// CTA, several CTAs per SM), both operands leave it through transposing ldmatrix loads (S^T is the MMA's A, X its
// B) and warp w multiplies into columns 16w..16w+15.  The row slices of one column tile form a thread-block
// cluster: every CTA leaves its partial tile in its own shared memory, and after a cluster barrier CTA q adds
// share q of the tile over all CTAs in rank order through distributed shared memory and stores it - no atomics,
// the same bits every time.  One launch serves both gradients: the first `tiles_a` column tiles take
// (v, x) -> dA, the others (u, dy) -> dB.
struct LoraGradPart {
  const __half* S;      // [M, 64]
  const __half* X;      // [M, C]
  float* out;           // [r, C], or [C, r] when `transposed`
  int C, transposed;
};
constexpr int LG_WARPS = 8, LG_THREADS = LG_WARPS * 32, LG_CT = 128, LG_RS = 32, LG_NS = 3;
constexpr int LG_XPITCH = LG_CT * 2 + 16, LG_SPITCH = 64 * 2 + 16;                   // bytes; +16 keeps ldmatrix rows on different banks
constexpr int LG_STAGE = LG_RS * (LG_XPITCH + LG_SPITCH);                            // 13312

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)) : "memory");
}
template <int R16>                               // r rounded up to sixteens: 1, 2 or 4
__global__ void __launch_bounds__(LG_THREADS)
lora_grads_kernel(const LoraGradPart pa, const LoraGradPart pb, int tiles_a, int M, int r, int rows_per_cta) {
  constexpr int RED_BYTES = R16 * 16 * LG_CT * 4;                                    // the partial tile, fp32 [16 R16][128]
  constexpr int SMEM = LG_NS * LG_STAGE > RED_BYTES ? LG_NS * LG_STAGE : RED_BYTES;
  __shared__ __align__(128) unsigned char smem[SMEM];
  const bool first = (int)blockIdx.x < tiles_a;
  const LoraGradPart& p = first ? pa : pb;
  const int c0 = (first ? blockIdx.x : blockIdx.x - tiles_a) * LG_CT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int C = p.C;
  const int m_begin = blockIdx.y * rows_per_cta, m_end = min(M, m_begin + rows_per_cta);
  const int n_it = m_end > m_begin ? (m_end - m_begin + LG_RS - 1) / LG_RS : 0;

  auto load_stage = [&](int it) {
    unsigned char* xs = smem + (it % LG_NS) * LG_STAGE;
    unsigned char* ss = xs + LG_RS * LG_XPITCH;
    const int m0 = m_begin + it * LG_RS;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int idx = threadIdx.x + q * LG_THREADS, row = idx >> 4, ch = idx & 15;
      const bool ok = m0 + row < m_end && c0 + 8 * ch < C;
      cp_async16_zfill(xs + row * LG_XPITCH + 16 * ch, p.X + (size_t)(ok ? m0 + row : 0) * C + (ok ? c0 + 8 * ch : 0), ok);
    }
    {
      const int row = threadIdx.x >> 3, ch = threadIdx.x & 7;
      const bool ok = m0 + row < m_end;
      cp_async16_zfill(ss + row * LG_SPITCH + 16 * ch, p.S + (size_t)(ok ? m0 + row : 0) * 64 + 8 * ch, ok);
    }
  };

  float acc[R16][2][4];
#pragma unroll
  for (int mt = 0; mt < R16; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

#pragma unroll
  for (int s = 0; s < LG_NS - 1; ++s) {
    if (s < n_it) load_stage(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const int mi = lane >> 3, rr = lane & 7;
  for (int it = 0; it < n_it; ++it) {
    asm volatile("cp.async.wait_group %0;" ::"n"(LG_NS - 2) : "memory");
    __syncthreads();                             // stage `it` has landed for everyone; stage it - 1 is free
    if (it + LG_NS - 1 < n_it) load_stage(it + LG_NS - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const unsigned char* xs = smem + (it % LG_NS) * LG_STAGE;
    const unsigned char* ss = xs + LG_RS * LG_XPITCH;
#pragma unroll
    for (int ks = 0; ks < LG_RS / 16; ++ks) {
      uint32_t b[4];                             // (k 0..7, n-tile 0), (k 8..15, n-tile 0), (k 0..7, n-tile 1), (k 8..15, n-tile 1)
      ldmatrix_x4_trans(b, xs + (ks * 16 + (mi & 1) * 8 + rr) * LG_XPITCH + 2 * (16 * warp + (mi >> 1) * 8));
#pragma unroll
      for (int mt = 0; mt < R16; ++mt) {
        uint32_t a[4];                           // (j 0..7, k 0..7), (j 8..15, k 0..7), (j 0..7, k 8..15), (j 8..15, k 8..15)
        ldmatrix_x4_trans(a, ss + (ks * 16 + (mi >> 1) * 8 + rr) * LG_SPITCH + 2 * (16 * mt + (mi & 1) * 8));
        mma_f16_16816(acc[mt][0], a[0], a[1], a[2], a[3], b[0], b[1]);
        mma_f16_16816(acc[mt][1], a[0], a[1], a[2], a[3], b[2], b[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                               // the ring is dead: its memory now holds the partial tile

  float* red = reinterpret_cast<float*>(smem);   // [16 R16][128]
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int mt = 0; mt < R16; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int col = 16 * warp + 8 * nt + 2 * t;
      red[(16 * mt + g) * LG_CT + col] = acc[mt][nt][0];
      red[(16 * mt + g) * LG_CT + col + 1] = acc[mt][nt][1];
      red[(16 * mt + g + 8) * LG_CT + col] = acc[mt][nt][2];
      red[(16 * mt + g + 8) * LG_CT + col + 1] = acc[mt][nt][3];
    }
  cluster_sync_all();
  const uint32_t rank = cluster_ctarank(), n_ranks = cluster_nctarank();
  const int total = r * LG_CT;                   // rows j < r only
  for (int idx = rank * LG_THREADS + threadIdx.x; idx < total; idx += n_ranks * LG_THREADS) {
    float s = 0.f;
    for (uint32_t q = 0; q < n_ranks; ++q) s += ld_dsmem_f32(red + idx, q);
    const int j = idx / LG_CT, c = c0 + (idx % LG_CT);
    if (c < C) {
      if (p.transposed) p.out[(size_t)c * r + j] = s;
      else p.out[(size_t)j * C + c] = s;
    }
  }
  cluster_sync_all();                            // nobody leaves while its tile is still being read
}

}  // namespace q4

using namespace q4;

extern "C" int q4_lora_project(const void* x, const void* w, void* out, int M, int C, int r, float scale, q4_stream_t stream) {
  if (!x || !w || !out) return fail(Q4_E_BADARG, "lora_project: null pointer");
  if (M <= 0 || C <= 0 || r < 1 || r > 64) return fail(Q4_E_BADARG, "lora_project: M=%d C=%d r=%d (1 <= r <= 64)", M, C, r);
  if (C % 32) return fail(Q4_E_SHAPE, "lora_project: the contraction length %d must be a multiple of 32", C);
  if (!aligned16(x) || !aligned16(w) || !aligned16(out)) return fail(Q4_E_ALIGN, "lora_project: pointers must be 16-byte aligned");
  if (int e = check_device()) return e;
  const int grid = (M + LP_ROWS - 1) / LP_ROWS;
  const cudaStream_t st = (cudaStream_t)stream;
  const __half *xh = (const __half*)x, *wh = (const __half*)w;
  __half* oh = (__half*)out;
  static std::atomic<bool> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev].load(std::memory_order_acquire)) {
    if (int e = check_cuda(cudaFuncSetAttribute(lora_project_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lora_project_smem<4>()), "lora_project smem attribute")) return e;
    if (int e = check_cuda(cudaFuncSetAttribute(lora_project_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lora_project_smem<8>()), "lora_project smem attribute")) return e;
    if (int e = check_cuda(cudaFuncSetAttribute(lora_project_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lora_project_smem<2>()), "lora_project smem attribute")) return e;
    if (int e = check_cuda(cudaFuncSetAttribute(lora_project_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lora_project_smem<1>()), "lora_project smem attribute")) return e;
    if (dev >= 0 && dev < 64) attr_done[dev].store(true, std::memory_order_release);
  }
  switch ((r + 7) / 8) {
    case 1: lora_project_kernel<1><<<grid, LP_THREADS, lora_project_smem<1>(), st>>>(xh, wh, oh, M, C, r, scale); break;
    case 2: lora_project_kernel<2><<<grid, LP_THREADS, lora_project_smem<2>(), st>>>(xh, wh, oh, M, C, r, scale); break;
    case 3: case 4: lora_project_kernel<4><<<grid, LP_THREADS, lora_project_smem<4>(), st>>>(xh, wh, oh, M, C, r, scale); break;
    default: lora_project_kernel<8><<<grid, LP_THREADS, lora_project_smem<8>(), st>>>(xh, wh, oh, M, C, r, scale); break;
  }
  return check_cuda(cudaGetLastError(), "lora_project launch");
}

extern "C" int q4_lora_grads(const void* v, const void* x, float* d_a, int K, const void* dy, const void* u, float* d_b, int N,
                             int M, int r, q4_stream_t stream) {
  const bool want_a = d_a != nullptr, want_b = d_b != nullptr;
  if (!want_a && !want_b) return Q4_OK;
  if (M <= 0 || r < 1 || r > 64) return fail(Q4_E_BADARG, "lora_grads: M=%d r=%d (1 <= r <= 64)", M, r);
  if (want_a && (!v || !x || K <= 0)) return fail(Q4_E_BADARG, "lora_grads: d_a needs v, x and K");
  if (want_b && (!u || !dy || N <= 0)) return fail(Q4_E_BADARG, "lora_grads: d_b needs u, dy and N");
  if ((want_a && K % 32) || (want_b && N % 32)) return fail(Q4_E_SHAPE, "lora_grads: K=%d and N=%d must be multiples of 32", K, N);
  if ((want_a && (!aligned16(v) || !aligned16(x))) || (want_b && (!aligned16(u) || !aligned16(dy))))
    return fail(Q4_E_ALIGN, "lora_grads: operands must be 16-byte aligned");
  if (int e = check_device()) return e;
  LoraGradPart pa{(const __half*)v, (const __half*)x, d_a, K, 0}, pb{(const __half*)u, (const __half*)dy, d_b, N, 1};
  const int tiles_a = want_a ? (K + LG_CT - 1) / LG_CT : 0, tiles_b = want_b ? (N + LG_CT - 1) / LG_CT : 0;
  // row slices per column tile (= CTAs per cluster): enough CTAs for two per SM, at least two stages of rows each
  int split = 1;
  while (split < 8 && (tiles_a + tiles_b) * split < 2 * sm_count() && M >= 4 * LG_RS * split) split *= 2;
  int rows_per_cta = ((M + split - 1) / split + LG_RS - 1) / LG_RS * LG_RS;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = (unsigned)split; at[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3((unsigned)(tiles_a + tiles_b), (unsigned)split); cfg.blockDim = dim3(LG_THREADS);
  cfg.dynamicSmemBytes = 0; cfg.stream = (cudaStream_t)stream; cfg.attrs = at; cfg.numAttrs = 1;
  cudaError_t le;
  switch ((r + 15) / 16) {
    case 1: le = cudaLaunchKernelEx(&cfg, lora_grads_kernel<1>, pa, pb, tiles_a, M, r, rows_per_cta); break;
    case 2: le = cudaLaunchKernelEx(&cfg, lora_grads_kernel<2>, pa, pb, tiles_a, M, r, rows_per_cta); break;
    default: le = cudaLaunchKernelEx(&cfg, lora_grads_kernel<4>, pa, pb, tiles_a, M, r, rows_per_cta); break;
  }
  if (le != cudaSuccess) return check_cuda(le, "lora_grads launch");
  return check_cuda(cudaGetLastError(), "lora_grads launch");
}
