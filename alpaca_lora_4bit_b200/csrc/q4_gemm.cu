// Large-M products over a packed int4 layer without materialising W in global memory:
//   forward   y [M, N] = x  [M, K] * W        (AutogradMatmul4bit forward,  autograd_4bit.py:34-43)
//   backward  dx[M, K] = dy [M, N] * W^T      (AutogradMatmul4bit backward, autograd_4bit.py:45-54)
// The reference reconstructs W into a dense fp16 [K, N] buffer and calls cuBLAS
// (matmul_utils_4bit.py:114-127).  Here each CTA dequantises the tiles of W it needs straight into
// shared memory, bit-exactly as the reference reconstruct does (rn(rn(s*q) - rn(s*(z+1)))), in
// the layout the 5th-generation tensor core reads, and tcgen05.mma accumulates in TMEM.
//
// Two kernels share the dequant routine and the operand layout.  The CTA-pair kernel (q4_gemm2.cuh)
// serves layers whose number of output columns is a multiple of 256; the single-CTA kernel in this
// file serves the rest (multiples of 128).  In the single-CTA kernel one CTA computes a 256 x 128
// output tile as two 128-row accumulators, so that every dequantised tile of W feeds two MMAs.
// Roles (320 threads):
//   warp 0      TMA producer: activation tiles [256 rows x 64 contraction] fp16, 128B-swizzled
//   warp 1      owns TMEM (256 fp32 columns) and issues tcgen05.mma (one elected thread)
//   warps 2-9   two groups of four: group 0 dequantises W for the even stages, group 1 for the
//               odd ones (packed words prefetched one own stage ahead); afterwards all eight run
//               the epilogue, one TMEM lane quarter of one accumulator each:
//               tcgen05.ld -> (+bias) -> fp16 -> global
// A stage holds 32 KiB of activations and 16 KiB of dequantised W:
//   forward   B = W[k0:k0+64, n0:n0+128], two panels of [64 k-rows][64 n = 128 B], MN-major operand
//   backward  B = W[k0:k0+128, n0:n0+64], one panel of [128 k-rows][64 n = 128 B], K-major operand
// Both are the same bytes: rows of 64 consecutive n for one k, 16-byte chunks XOR-swizzled with
// the row index (the 128B swizzle pattern), so one dequant routine serves both directions: a
// thread takes 8 packed words (8 k-rows x 8 columns) and writes eight 16-byte chunks.
// Scales and rn(s*(z+1)) come from shared-memory tables (forward: all groups x the CTA's 128
// columns, built once) or, in the backward, from global memory per row with reuse while the group
// stays the same.  Act-order is free in this scheme: the group of every row is read from g_idx.
// Every mbarrier wait is bounded: on expiry the kernel records a status word and stops waiting.
#include "q4_umma.cuh"

namespace q4 {

__device__ unsigned g_gemm_status = 0;        // Q4_STATUS_WAIT_EXPIRED if any bounded wait gave up

constexpr int GM_TILE_M = 256;                // two accumulators of 128 rows
constexpr int GM_TILE_N = 128;                // output columns per CTA
constexpr int GM_TILE_C = 64;                 // contraction elements per stage
constexpr int GM_MAX_STAGES = 4;
constexpr int GM_A_BYTES = GM_TILE_M * GM_TILE_C * 2;     // 32 KiB
constexpr int GM_B_BYTES = 128 * 64 * 2;                  // 16 KiB
constexpr int GM_STAGE_BYTES = GM_A_BYTES + GM_B_BYTES;
constexpr int GM_THREADS = 320;
constexpr int GM_DEQ_THREADS = 128;           // per dequant group
constexpr int GM_DEQ_GROUPS = 2;
constexpr int GM_TMEM_COLS = 256;
constexpr uint32_t GM_WAIT_TRIES = 40000;     // x ~2 us sleeping tries
constexpr size_t Q4_GEMM_WS_COUNTER_BYTES = 65536;          // head of the workspace: arrival counters
constexpr size_t Q4_GEMM_WS_SLICE_BYTES = 256 * 256 * 4;    // fp32 partial sums of one slice of one 256 x 256 tile

struct GemmParams {
  const uint32_t* qw;       // [K/8, N]
  const __half* scales;     // [G, N]
  const uint32_t* qzeros;   // [G, N/8]
  const int* g_idx;         // [K]
  const __half* bias;       // [N_out] or null (forward only)
  const __half* residual;   // [M, N_out] added to the output, or null (forward only)
  __half* out;              // [M, N_out]
  int M, K, N, G;
  int n_contract_tiles;     // contraction length / 64
  int stages;               // pipeline depth (3 or 4, what shared memory allows)
  unsigned long long* trace;  // optional per-CTA cycle trace (256 slots), else null
  // Optional low-rank term added through one extra pipeline stage (null / 0 = none):
  //   forward   y  += U * lora_B^T,  U = scale * x  * lora_A^T  [M, 64] (zero-padded),  lora_w = lora_B [N, r]
  //   backward  dx += V * lora_A,    V = scale * dy * lora_B    [M, 64] (zero-padded),  lora_w = lora_A [r, K]
  const __half* lora_w;
  int lora_r;
  // CTA-pair kernel, when tiles x contraction stages are dealt to the pairs as one sequence: fp32
  // partial sums of shared tiles ([pair][256 or 512 x 256]) and one arrival counter per 32 rows of a
  // shared tile (indexed by the first contributing pair), zero between launches.
  float* ws_partials;
  unsigned* ws_counters;
  const __half* zp_table;   // rn(s * (z+1)) for every [group, column], or null
  int seq_shift;            // > 0: the caller promises g_idx[k] == k >> seq_shift (sequential groups of 2^seq_shift rows)
};

__device__ __forceinline__ void gm_mark(unsigned long long* tr, int slot) {
  if (tr && slot < 256) tr[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 256 + slot] = clock64();
}

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;        // the common case once the pipeline is full
  const uint32_t lim = *abort_flag ? 4u : GM_WAIT_TRIES;
  for (uint32_t i = 0; i < lim; ++i)
    if (mbar_try_wait_sleep(bar, parity, 2000u)) return true;
  *abort_flag = 1;
  atomicExch(&g_gemm_status, Q4_STATUS_WAIT_EXPIRED);
  return false;
}

template <bool TRANSPOSE>
__global__ void __launch_bounds__(GM_THREADS, 1)
q4_gemm_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap umap, const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);      // 1024-byte aligned, still a shared-space pointer
  unsigned char* stages = smem;
  const int S = p.stages;
  uint64_t* full_a = reinterpret_cast<uint64_t*>(smem + S * GM_STAGE_BYTES);
  uint64_t* full_b = full_a + GM_MAX_STAGES;
  uint64_t* empty = full_b + GM_MAX_STAGES;
  uint64_t* acc_full = empty + GM_MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // forward: [G][128 scales | 128 rn(s*(z+1))], 512 bytes per group
  unsigned char* tab = smem + S * GM_STAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int out0 = blockIdx.x * GM_TILE_N;            // first output column (n forward, k backward)
  const int m0 = blockIdx.y * GM_TILE_M;
  const int T = p.n_contract_tiles;
  const int TT = T + (p.lora_r > 0 ? 1 : 0);          // one more stage for the low-rank term
  const int lora_ks = (p.lora_r + 15) >> 4;           // its 16-wide MMA steps

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(&full_a[i], 1); mbar_init(&full_b[i], GM_DEQ_THREADS / 32); mbar_init(&empty[i], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&amap);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, GM_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: activation tiles ----------------
    if (lane == 0) {
      for (int it = 0; it < TT; ++it) {
        const int st = it % S, use = it / S;
        if (use > 0) wait_bar(&empty[st], (use - 1) & 1, abort_flag);
        mbar_arrive_expect_tx(&full_a[st], GM_A_BYTES);
        if (it < T) tma_load_2d(stages + (size_t)st * GM_STAGE_BYTES, &amap, it * GM_TILE_C, m0, &full_a[st]);
        else tma_load_2d(stages + (size_t)st * GM_STAGE_BYTES, &umap, 0, m0, &full_a[st]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(128, GM_TILE_N, !TRANSPOSE);
      for (int it = 0; it < TT; ++it) {
        const int st = it % S, use = it / S;
        const int nks = it < T ? GM_TILE_C / 16 : lora_ks;
        if (it < 20) gm_mark(p.trace, 3 * it);
        wait_bar(&full_a[st], use & 1, abort_flag);
        if (it < 20) gm_mark(p.trace, 3 * it + 1);
        wait_bar(&full_b[st], use & 1, abort_flag);
        if (it < 20) gm_mark(p.trace, 3 * it + 2);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(stages + (size_t)st * GM_STAGE_BYTES);
        const uint32_t b_addr = a_addr + GM_A_BYTES;
#pragma unroll
        for (int ks = 0; ks < GM_TILE_C / 16; ++ks) {
          if (ks >= nks) break;
          // A: K-major, 128-byte rows, 8-row groups 1024 B apart; 16 contraction elements = 32 B
          const uint64_t ad0 = smem_desc_sw128(a_addr + ks * 32, 16, 1024);
          const uint64_t ad1 = smem_desc_sw128(a_addr + GM_A_BYTES / 2 + ks * 32, 16, 1024);      // rows 128..255
          // forward  B: MN-major: 64 n contiguous (128 B) per k-row, next 64 n at +8192, next 8 k-rows at +1024
          // backward B: K-major like A
          const uint64_t bd = TRANSPOSE ? smem_desc_sw128(b_addr + ks * 32, 16, 1024)
                                        : smem_desc_sw128(b_addr + ks * 2048, 8192, 1024);
          umma_f16(tmem_acc, ad0, bd, idesc, (it > 0 || ks > 0) ? 1u : 0u);
          umma_f16(tmem_acc + 128, ad1, bd, idesc, (it > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&empty[st]);                   // frees the stage when these MMAs have read it
      }
      umma_commit(acc_full);
    }
  } else {
    // ---------------- dequantisers (then epilogue) ----------------
    const int grp = (warp - 2) >> 2;                               // dequant group: stages it % 2 == grp
    const int tid = (threadIdx.x - 64) & (GM_DEQ_THREADS - 1);     // 0..127 within the group
    const int chunk16 = TRANSPOSE ? (tid & 7) : (tid & 15);        // 16-byte chunk (8 columns) within the stage's n-range
    const int r = TRANSPOSE ? (tid >> 3) : (tid >> 4);             // packed row within the stage
    const int N = p.N;
    uint32_t off[8];
    deq_offsets(chunk16 & 7, off);
    if (!TRANSPOSE) {
      // tables for the CTA's 128 columns: scale and rn(s*(z+1)) of every group
      for (int i = threadIdx.x - 64; i < p.G * (GM_TILE_N / 8); i += GM_DEQ_THREADS * GM_DEQ_GROUPS) {
        const int g = i / (GM_TILE_N / 8), c8 = i % (GM_TILE_N / 8);
        const uint4 s = __ldg(reinterpret_cast<const uint4*>(p.scales + (size_t)g * N + out0 + 8 * c8));
        const uint32_t zw = __ldg(p.qzeros + (size_t)g * (N >> 3) + ((out0 + 8 * c8) >> 3));
        const uint4 z = zero_terms(s, zw);
        *reinterpret_cast<uint4*>(tab + g * 512 + 16 * c8) = s;
        *reinterpret_cast<uint4*>(tab + g * 512 + 256 + 16 * c8) = z;
      }
      named_bar_sync(1, GM_DEQ_THREADS * GM_DEQ_GROUPS);
    }
    // packed words of the stage: rows (k0/8 + r), columns ncol0 .. ncol0+7
    auto word_ptr = [&](int it) -> const uint32_t* {
      const int prow = TRANSPOSE ? (out0 >> 3) + r : it * (GM_TILE_C >> 3) + r;
      const int ncol = TRANSPOSE ? it * GM_TILE_C + 8 * chunk16 : out0 + 8 * chunk16;
      return p.qw + (size_t)prow * N + ncol;
    };
    uint4 wa = make_uint4(0, 0, 0, 0), wb = wa;
    int4 ga = make_int4(0, 0, 0, 0), gb = ga;                      // groups of the task's 8 k-rows
    if (grp < T) {
      wa = ldg_stream(word_ptr(grp)); wb = ldg_stream(word_ptr(grp) + 4);
      const int k8 = TRANSPOSE ? out0 + 8 * r : grp * GM_TILE_C + 8 * r;
      ga = __ldg(reinterpret_cast<const int4*>(p.g_idx + k8));
      gb = __ldg(reinterpret_cast<const int4*>(p.g_idx + k8 + 4));
    }
    for (int it = grp; it < TT; it += GM_DEQ_GROUPS) {
      const int st = it % S, use = it / S;
      if (it == T) {
        // ---- low-rank stage: B operand from lora_w instead of dequantised weights ----
        if (use > 0 && lane == 0) wait_bar(&empty[st], (use - 1) & 1, abort_flag);
        __syncwarp();
        unsigned char* bst = stages + (size_t)st * GM_STAGE_BYTES + GM_A_BYTES;
        const int rr = p.lora_r, rows = 16 * lora_ks;
        if (!TRANSPOSE) {
          // column n = out0 + tid: element (j, n) = lora_B[n][j] into panel tid/64, row j, 128B-swizzled
          const __half* src = p.lora_w + (size_t)(out0 + tid) * rr;
          unsigned char* col = bst + (tid >> 6) * 8192 + ((tid & 7) << 1);
          const int cc = (tid & 63) >> 3;
          for (int j = 0; j < rows; ++j) {
            const __half v = j < rr ? src[j] : __float2half(0.f);
            *reinterpret_cast<__half*>(col + j * 128 + ((cc ^ (j & 7)) << 4)) = v;
          }
        } else {
          // row k = out0 + tid: element (k, j) = lora_A[j][k], 8 j per 16-byte chunk
          unsigned char* row = bst + tid * 128;
          for (int c8 = 0; c8 < 2 * lora_ks; ++c8) {
            uint4 o;
            __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int j = 8 * c8 + e;
              oh[e] = j < rr ? p.lora_w[(size_t)j * p.K + out0 + tid] : __float2half(0.f);
            }
            *reinterpret_cast<uint4*>(row + ((c8 ^ (tid & 7)) << 4)) = o;
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_b[st]);
        continue;
      }
      const uint32_t w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
      const int gi[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
      if (it + GM_DEQ_GROUPS < T) {                                // prefetch this group's next stage
        wa = ldg_stream(word_ptr(it + GM_DEQ_GROUPS)); wb = ldg_stream(word_ptr(it + GM_DEQ_GROUPS) + 4);
        if (!TRANSPOSE) {
          const int k8 = (it + GM_DEQ_GROUPS) * GM_TILE_C + 8 * r;
          ga = __ldg(reinterpret_cast<const int4*>(p.g_idx + k8));
          gb = __ldg(reinterpret_cast<const int4*>(p.g_idx + k8 + 4));
        }
      }
      if (threadIdx.x == 64 && it < 40) gm_mark(p.trace, 64 + 3 * (it / 2));
      if (use > 0 && lane == 0) wait_bar(&empty[st], (use - 1) & 1, abort_flag);
      __syncwarp();
      if (threadIdx.x == 64 && it < 40) gm_mark(p.trace, 65 + 3 * (it / 2));
      unsigned char* bst = stages + (size_t)st * GM_STAGE_BYTES + GM_A_BYTES;
      // forward: panel (chunk16 / 8) of [64 rows][128 B]; backward: one panel of [128 rows][128 B]
      unsigned char* rows8 = bst + (TRANSPOSE ? r * 1024 : (chunk16 >> 3) * 8192 + r * 1024);
      const int4 ga_now = make_int4(gi[0], gi[1], gi[2], gi[3]), gb_now = make_int4(gi[4], gi[5], gi[6], gi[7]);
      if (TRANSPOSE) {
        const int ncol = it * GM_TILE_C + 8 * chunk16;             // global column of the task
        deq_task_global(rows8, off, w, ga_now, gb_now, p.scales + ncol, p.qzeros + (ncol >> 3), N);
      } else {
        deq_task_tables(rows8, off, w, ga_now, gb_now, tab + 16 * chunk16);
      }
      fence_async_smem();                          // generic-proxy stores -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_b[st]);
      if (threadIdx.x == 64 && it < 40) gm_mark(p.trace, 66 + 3 * (it / 2));
    }
    if (threadIdx.x == 64) gm_mark(p.trace, 200);

    // ---------------- epilogue: TMEM -> registers -> fp16 -> global ----------------
    if (lane == 0) wait_bar(acc_full, 0, abort_flag);
    __syncwarp();
    tc_fence_after();
    const int quarter = warp & 3;                                  // TMEM lanes 32*quarter .. +31
    const int half = grp;                                          // accumulator (rows 128*half ..)
    const int m = m0 + 128 * half + 32 * quarter + lane;
    const int n_out_total = TRANSPOSE ? p.K : p.N;
#pragma unroll 1
    for (int cb = 0; cb < GM_TILE_N / 32; ++cb) {
      uint32_t v[32];
      __syncwarp();                                // the lanes of rows past M skipped the stores: whole again for the warp-wide load
      tmem_ld32(tmem_acc + ((uint32_t)(32 * quarter) << 16) + 128 * half + cb * 32, v);
      tmem_ld_wait();
      if (m < p.M) {
        __half* dst = p.out + (size_t)m * n_out_total + out0 + cb * 32;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float f0 = __uint_as_float(v[8 * q + 2 * e]), f1 = __uint_as_float(v[8 * q + 2 * e + 1]);
            if (!TRANSPOSE && p.bias) {
              f0 += __half2float(p.bias[out0 + cb * 32 + 8 * q + 2 * e]);
              f1 += __half2float(p.bias[out0 + cb * 32 + 8 * q + 2 * e + 1]);
            }
            __half2 hv = __floats2half2_rn(f0, f1);
            if (!TRANSPOSE && p.residual) {              // rounded first, as the separate add of the decoder layer would see it
              const float2 rr = __half22float2(*reinterpret_cast<const __half2*>(p.residual + (size_t)m * n_out_total + out0 + cb * 32 + 8 * q + 2 * e));
              const float2 yy = __half22float2(hv);
              hv = __floats2half2_rn(yy.x + rr.x, yy.y + rr.y);
            }
            ov[e] = as_u32(hv);
          }
          *reinterpret_cast<uint4*>(dst + 8 * q) = o;
        }
      }
    }
  }
  if (threadIdx.x == 64) gm_mark(p.trace, 201);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_acc, GM_TMEM_COLS);
}

static unsigned long long* g_gemm_trace = nullptr;

// rn(s * (z+1)) of every [group, column]: what the backward would otherwise recompute for every
// row of every task when the rows of a task belong to different groups (act-order).
__global__ void zp_table_kernel(const __half* __restrict__ scales, const uint32_t* __restrict__ qzeros, __half* __restrict__ out, int total8) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  const uint4 s = __ldg(reinterpret_cast<const uint4*>(scales) + i);
  reinterpret_cast<uint4*>(out)[i] = zero_terms(s, __ldg(qzeros + i));
}

static int g_gemm_variant = 0;                // 0 = choose per shape, 1 = single-CTA kernel, 2 = CTA-pair kernel with 256-row tiles,
                                              // 3 = CTA-pair kernel with 512-row tiles, 4 = weights-in-TMEM kernel (forward,
                                              // sequential groups promised), 5 = as 0 but never the weights-in-TMEM kernel

static size_t gemm_smem_bytes(bool transpose, int G, int stages) {
  return 1024 + (size_t)stages * GM_STAGE_BYTES + 256 + (transpose ? 0 : (size_t)2 * G * GM_TILE_N * sizeof(__half));
}

}  // namespace q4

#include "q4_gemm2.cuh"
#include "q4_gemm3.cuh"

using namespace q4;

// Estimated duration (SM cycles) of the pair kernel with tiles of 256 * mh rows, and whether that
// assumes whole tiles per pair (round after round) or all tiles x stages dealt as one sequence.
// Per contraction stage a pair takes about 700 cycles with 256-row tiles (bounded by the dequant
// warps) and 1100 with 512-row tiles (bounded by the MMAs: twice the flops per stage); exchanging
// the partial sums of a shared tile costs about as much as 12 resp. 16 stages.
static long long gemm2_estimate(int M, int nout, int T, int P, int mh, bool ws_ok, bool* stream) {
  const int tile_m = 256 * mh;
  const long long n_tiles = (long long)(nout / G2_TILE_N) * ((M + tile_m - 1) / tile_m);
  const long long per_stage = mh == 2 ? 1100 : 700, exchange = mh == 2 ? 16 : 12;
  long long best = (n_tiles + P - 1) / P * T;
  *stream = false;
  if (ws_ok && T >= 8 && n_tiles % P != 0) {
    const long long total = n_tiles * T, dealt = (total + P - 1) / P + exchange;
    if (dealt < best && total >= (long long)P * 4 && total * P < (1ll << 32)) { best = dealt; *stream = true; }
  }
  return best * per_stage;
}

static int gemm_launch(bool transpose, const void* act, const int32_t* qweight, void* out, const void* scales,
                       const int32_t* qzeros, const int32_t* g_idx, const void* bias, const void* lora_u,
                       const void* lora_w, int lora_r, int M, int K, int N, int G, void* workspace, size_t workspace_bytes,
                       q4_stream_t stream, bool swiglu = false, const void* zp_cached = nullptr, const void* residual = nullptr,
                       int seq_groupsize = 0) {
  if (!act || !qweight || !out || !scales || !qzeros || !g_idx) return fail(Q4_E_BADARG, "gemm: null pointer");
  const int gv = g_gemm_variant == 5 ? 0 : g_gemm_variant;
  if (M <= 0 || K <= 0 || N <= 0 || G <= 0) return fail(Q4_E_BADARG, "gemm: M=%d K=%d N=%d G=%d", M, K, N, G);
  if (K % 128 || N % 128) return fail(Q4_E_SHAPE, "gemm: K=%d and N=%d must be multiples of 128", K, N);
  if (!aligned16(act) || !aligned16(qweight) || !aligned16(out) || !aligned16(scales) || !aligned16(g_idx))
    return fail(Q4_E_ALIGN, "gemm: pointers must be 16-byte aligned");
  if (lora_r < 0 || lora_r > 64) return fail(Q4_E_SHAPE, "gemm: low-rank width %d outside 0..64", lora_r);
  if (lora_r > 0 && (!lora_u || !lora_w || !aligned16(lora_u) || !aligned16(lora_w)))
    return fail(Q4_E_BADARG, "gemm: the low-rank term needs 16-byte aligned lora_u [M,64] and lora_w");
  if (workspace && !aligned16(workspace)) return fail(Q4_E_ALIGN, "gemm: the workspace must be 16-byte aligned");
  if (residual && (transpose || swiglu || !aligned16(residual))) return fail(Q4_E_BADARG, "gemm: a residual needs the plain forward and 16-byte alignment");
  if (int e = check_device()) return e;
  const int contract = transpose ? N : K, nout = transpose ? K : N;
  // forward with the caller's zero-term table: scales and zero terms come from L2 as in the backward, and the
  // shared memory the tables would take goes to pipeline stages (CTA-pair kernel only)
  const bool may_drop_tables = !transpose && zp_cached != nullptr;
  int stages2 = gemm2_stages(transpose, G, 1), stages2w = gemm2_stages(transpose, G, 2);
  const int stages2_nt = may_drop_tables ? gemm2_stages(true, G, 1) : stages2, stages2w_nt = may_drop_tables ? gemm2_stages(true, G, 2) : stages2w;
  // the table is used where it buys a stage for both tile heights (or makes the pair kernel possible at all)
  // groups promised sequential (a power of two of at least 8 rows): the forward fetches a task's scales and zero terms
  // one task ahead with its packed words, so the table is taken whether or not it buys a stage
  int seq_shift = 0;
  if (seq_groupsize >= 8 && (seq_groupsize & (seq_groupsize - 1)) == 0 && (long long)seq_groupsize * G >= K)
    while ((1 << seq_shift) < seq_groupsize) ++seq_shift;
  const bool no_tables = transpose || (may_drop_tables && ((stages2_nt > stages2 && stages2w_nt > stages2w) || seq_shift > 0));
  if (no_tables && !transpose) { stages2 = stages2_nt; stages2w = stages2w_nt; }
  const bool pair_ok = nout % G2_TILE_N == 0 && stages2 > 0;
  const bool wide_ok = nout % G2_TILE_N == 0 && stages2w > 0;
  if ((gv == 2 && !pair_ok) || (gv == 3 && !wide_ok))
    return fail(Q4_E_SHAPE, "gemm: the CTA-pair kernel needs %d output columns to be a multiple of 256 and G=%d tables to fit", nout, G);
  if (swiglu && (transpose || lora_r > 0 || !pair_ok || N % 256))
    return fail(Q4_E_SHAPE, "gemm: the fused gate_up product needs the CTA-pair kernel (N=%d a multiple of 256, G=%d tables that fit) and no low-rank term", N, G);
  const bool use_pair = (pair_ok && gv != 1) || gv == 3 || swiglu;
  // weights-in-TMEM kernel: forward, groups of at least the 64 contraction elements of a stage promised sequential
  const bool tm_ok = !transpose && !swiglu && no_tables && seq_shift >= 6 && nout % G2_TILE_N == 0;
  if (gv == 4 && !tm_ok)
    return fail(Q4_E_SHAPE, "gemm: the weights-in-TMEM kernel takes the forward of a layer with N=%d a multiple of 256, its zero-term table and sequential groups of 64 rows or more", N);
  // 512-row tiles halve the dequant work per flop but leave fewer, larger tiles to deal: take the
  // form the estimate favours
  const int P_est = sm_count() / 2 > 0 ? sm_count() / 2 : 1;
  const size_t zp_need = transpose && !zp_cached ? (((size_t)G * N * sizeof(__half) + 255) & ~(size_t)255) : 0;
  auto ws_ok_for = [&](int m) { return workspace && workspace_bytes >= Q4_GEMM_WS_COUNTER_BYTES + zp_need + (size_t)P_est * m * Q4_GEMM_WS_SLICE_BYTES; };
  int mh = 1;
  if (use_pair && gv == 3) mh = 2;
  else if (use_pair && gv == 0 && wide_ok && M > 256) {
    bool s1, s2;
    const long long e1 = gemm2_estimate(M, nout, contract / GM_TILE_C, P_est, 1, ws_ok_for(1), &s1);
    const long long e2 = gemm2_estimate(M, nout, contract / GM_TILE_C, P_est, 2, ws_ok_for(2), &s2);
    if (e2 < e1) mh = 2;
  }
  // taken where the pair kernel would run 256-row tiles, where all its tiles fit one round, and up to 1024 rows (beyond,
  // 512-row tiles of the pair kernel - half the dequant work per flop - measured faster on the wide layers)
  const bool use_tm = tm_ok && use_pair &&
                      (gv == 4 || (gv == 0 && g_gemm_variant != 5 && (mh == 1 || M <= 1024 || (long long)(nout / G2_TILE_N) * ((M + 255) / 256) <= P_est)));
  if (use_tm) mh = 1;                          // its TMA boxes are 128 activation rows, as for 256-row tiles
  int stages = GM_MAX_STAGES;
  while (stages > 2 && gemm_smem_bytes(transpose, G, stages) > 227 * 1024) --stages;
  if (use_pair) stages = mh == 2 ? stages2w : stages2;
  const size_t smem = use_pair ? gemm2_smem_bytes(no_tables, G, stages, mh) : gemm_smem_bytes(transpose, G, stages);
  if (smem > 227 * 1024) return fail(Q4_E_SHAPE, "gemm: scale tables for G=%d groups do not fit shared memory", G);

  GemmParams p;
  p.qw = (const uint32_t*)qweight; p.scales = (const __half*)scales; p.qzeros = (const uint32_t*)qzeros;
  p.g_idx = g_idx; p.bias = (const __half*)bias; p.out = (__half*)out;
  p.residual = (!transpose && !swiglu) ? (const __half*)residual : nullptr;
  p.M = M; p.K = K; p.N = N; p.G = G;
  p.n_contract_tiles = contract / GM_TILE_C;
  p.stages = stages;
  p.trace = g_gemm_trace;
  p.lora_w = lora_r > 0 ? (const __half*)lora_w : nullptr;
  p.lora_r = lora_r;
  p.ws_partials = nullptr; p.ws_counters = nullptr; p.zp_table = nullptr;
  p.seq_shift = (!transpose && no_tables) ? seq_shift : 0;
  const int box_rows = use_pair ? 128 * mh : GM_TILE_M;    // activation rows one TMA copy brings
  CUtensorMap amap;
  if (int e = make_tmap_2d(&amap, act, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)contract, (uint64_t)M,
                           (uint64_t)contract * 2, GM_TILE_C, box_rows, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  CUtensorMap umap = amap;
  if (lora_r > 0)
    if (int e = make_tmap_2d(&umap, lora_u, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, 64, (uint64_t)M, 128, GM_TILE_C, box_rows,
                             CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  // once per device, direction and kernel: raise the dynamic shared memory limit to the largest the
  // kernel can ask for and, for the pair kernel, ask how many pairs can be resident at once
  static bool attr_done[2][2][64] = {{{false}}};
  static int max_pairs[2][64] = {{0}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  const int tr = transpose ? 1 : 0;
  if (!attr_done[use_pair ? 1 : 0][tr][dev]) {
    const int cap = 227 * 1024;
    const void* fn = use_pair ? (transpose ? (const void*)q4_gemm2_kernel<true, false, 1> : (const void*)q4_gemm2_kernel<false, false, 1>)
                              : (transpose ? (const void*)q4_gemm_kernel<true> : (const void*)q4_gemm_kernel<false>);
    if (int e = check_cuda(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, cap), "gemm smem attribute")) return e;
    if (use_pair) {
      const void* more[3] = {transpose ? (const void*)q4_gemm2_kernel<true, true, 1> : (const void*)q4_gemm2_kernel<false, true, 1>,
                             transpose ? (const void*)q4_gemm2_kernel<true, false, 2> : (const void*)q4_gemm2_kernel<false, false, 2>,
                             transpose ? (const void*)q4_gemm2_kernel<true, true, 2> : (const void*)q4_gemm2_kernel<false, true, 2>};
      for (const void* f2 : more)
        if (int e = check_cuda(cudaFuncSetAttribute(f2, cudaFuncAttributeMaxDynamicSharedMemorySize, cap), "gemm smem attribute")) return e;
    }
    if (use_pair) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * sm_count(), 1, 1); cfg.blockDim = dim3(G2_THREADS, 1, 1); cfg.dynamicSmemBytes = cap;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      int nc = 0;
      if (cudaOccupancyMaxActiveClusters(&nc, fn, &cfg) != cudaSuccess || nc <= 0) { cudaGetLastError(); nc = sm_count() / 2; }
      max_pairs[tr][dev] = nc;
    }
    attr_done[use_pair ? 1 : 0][tr][dev] = true;
  }
  static bool swiglu_attr_done[64] = {false};
  if (swiglu && !swiglu_attr_done[dev]) {
    const void* fns[4] = {(const void*)q4_gemm2_kernel<false, false, 1, true>, (const void*)q4_gemm2_kernel<false, true, 1, true>,
                          (const void*)q4_gemm2_kernel<false, false, 2, true>, (const void*)q4_gemm2_kernel<false, true, 2, true>};
    for (const void* f2 : fns)
      if (int e = check_cuda(cudaFuncSetAttribute(f2, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024), "gemm smem attribute")) return e;
    swiglu_attr_done[dev] = true;
  }
  if (use_pair) {
    const int tile_m = 256 * mh;
    const int n_tiles = (nout / G2_TILE_N) * ((M + tile_m - 1) / tile_m);
    const int P = max_pairs[tr][dev], T = p.n_contract_tiles;
    unsigned char* ws = (unsigned char*)workspace;
    size_t ws_off = Q4_GEMM_WS_COUNTER_BYTES;
    // backward: table of zero terms in the workspace, filled by a small kernel ahead of the GEMM
    p.zp_table = nullptr;
    const size_t zp_bytes = ((size_t)G * N * sizeof(__half) + 255) & ~(size_t)255;
    if (zp_cached && (transpose || no_tables)) {
      p.zp_table = (const __half*)zp_cached;                 // the caller keeps the table of this layer
    } else if (transpose && ws && workspace_bytes >= ws_off + zp_bytes) {
      p.zp_table = (const __half*)(ws + ws_off);
      const int total8 = G * (N / 8);
      zp_table_kernel<<<(total8 + 255) / 256, 256, 0, st>>>((const __half*)scales, (const uint32_t*)qzeros, (__half*)(ws + ws_off), total8);
      ws_off += zp_bytes;
    }
    if (use_tm) {
      static bool tm_attr_done[64] = {false};
      if (!tm_attr_done[dev]) {
        for (const void* f3 : {(const void*)q4_gemm3_kernel<false>, (const void*)q4_gemm3_kernel<true>})
          if (int e = check_cuda(cudaFuncSetAttribute(f3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm3_smem_bytes()), "gemm smem attribute")) return e;
        tm_attr_done[dev] = true;
      }
      // whole tiles round after round, or - where the last round would leave pairs idle for longer than the exchange
      // of partial sums costs - all tiles x stages as one sequence in equal runs (as for the pair kernel below)
      const int tiles3 = (nout / G2_TILE_N) * ((M + 255) / 256);
      int pairs3 = tiles3 < P ? tiles3 : P;
      bool stream3 = false;
      const long long total3 = (long long)tiles3 * T;
      // (measured: every further item of a pair's run and the exchange cost about 30 stages together; tiles cut
      // between several whole pairs - fewer tiles than pairs - never paid)
      if (ws && workspace_bytes >= ws_off + (size_t)P * Q4_GEMM_WS_SLICE_BYTES && T >= 8 && tiles3 > P && tiles3 % P != 0 &&
          total3 * P < (1ll << 32)) {
        const long long whole = (long long)((tiles3 + P - 1) / P) * T, dealt = (total3 + P - 1) / P + 30;
        stream3 = dealt < whole;
      }
      // Few tiles and a long contraction (short prompts: one row tile, 16 column tiles of a 4096-wide layer on 74
      // pairs): every tile is cut between a whole number of pairs.  The exchange costs about 12 + 7 nb stages (nb =
      // blocks of 32 rows a tile really has: the partial sums of the other rows are neither written nor read), so it
      // pays for short prompts and long contractions (64 rows at 4096 x 4096: 25.7 -> 18.4 us; 32 rows at 11008 x 4096:
      // 58.2 -> 24.8 us) and not at 256 rows of 4096 x 4096 (27.3 -> 32.8 us).
      if (!stream3 && ws && workspace_bytes >= ws_off + (size_t)P * Q4_GEMM_WS_SLICE_BYTES && tiles3 * 2 <= P && T >= 16) {
        int per_tile = P / tiles3;
        if (per_tile > T / 8) per_tile = T / 8;
        const int nb = ((M < 256 ? M : 256) + 31) / 32;
        if (per_tile >= 2 && (long long)T * (per_tile - 1) / per_tile > 12 + 7 * nb) { stream3 = true; pairs3 = tiles3 * per_tile; }
      }
      p.ws_partials = (float*)(ws + ws_off);
      p.ws_counters = (unsigned*)ws;
      if (stream3) q4_gemm3_kernel<true><<<dim3(2 * pairs3), dim3(G3_THREADS), gemm3_smem_bytes(), st>>>(amap, umap, p);
      else q4_gemm3_kernel<false><<<dim3(2 * pairs3), dim3(G3_THREADS), gemm3_smem_bytes(), st>>>(amap, umap, p);
      return check_cuda(cudaGetLastError(), "gemm launch");
    }
    // Whole tiles per pair, round after round - or, when the last round would leave pairs idle for
    // longer than the exchange of partial sums costs (about a dozen stages), all tiles x stages as one
    // sequence cut into equal runs.
    bool stream = false;
    int pairs = n_tiles < P ? n_tiles : P;
    gemm2_estimate(M, nout, T, P, mh, ws && workspace_bytes >= ws_off + (size_t)P * mh * Q4_GEMM_WS_SLICE_BYTES, &stream);
    if (stream) {
      // Fewer tiles than half the pairs: take a whole number of pairs per tile, so that every tile is shared by the
      // same number of pairs in equal parts and a pair has one piece of one tile.  Cut into P runs the pieces fall
      // anywhere, a pair's run can lie inside one tile, and the tile's reducer then waits for a contributor that ends
      // when it does (32 tiles x 172 stages at 1024 rows: 90.2 us on 74 pairs, 78.6 us on 64).
      const int per_tile = n_tiles > 0 ? P / n_tiles : 0;
      pairs = per_tile >= 2 ? n_tiles * per_tile : P;
    }
    const int f = stream ? 2 : 1;
    p.ws_partials = (float*)(ws + ws_off);
    p.ws_counters = (unsigned*)ws;
    const dim3 grid(2 * pairs), block(G2_THREADS);
#define Q4_LAUNCH2(TR, SP, MHV) q4_gemm2_kernel<TR, SP, MHV><<<grid, block, smem, st>>>(amap, umap, p)
#define Q4_LAUNCH2S(SP, MHV) q4_gemm2_kernel<false, SP, MHV, true><<<grid, block, smem, st>>>(amap, umap, p)
    if (swiglu) {
      if (mh == 2) { if (f > 1) Q4_LAUNCH2S(true, 2); else Q4_LAUNCH2S(false, 2); }
      else { if (f > 1) Q4_LAUNCH2S(true, 1); else Q4_LAUNCH2S(false, 1); }
    } else if (mh == 2) {
      if (f > 1) { if (transpose) Q4_LAUNCH2(true, true, 2); else Q4_LAUNCH2(false, true, 2); }
      else { if (transpose) Q4_LAUNCH2(true, false, 2); else Q4_LAUNCH2(false, false, 2); }
    } else {
      if (f > 1) { if (transpose) Q4_LAUNCH2(true, true, 1); else Q4_LAUNCH2(false, true, 1); }
      else { if (transpose) Q4_LAUNCH2(true, false, 1); else Q4_LAUNCH2(false, false, 1); }
    }
#undef Q4_LAUNCH2
#undef Q4_LAUNCH2S
  } else {
    const dim3 grid(nout / GM_TILE_N, (M + GM_TILE_M - 1) / GM_TILE_M), block(GM_THREADS);
    if (transpose) q4_gemm_kernel<true><<<grid, block, smem, st>>>(amap, umap, p);
    else q4_gemm_kernel<false><<<grid, block, smem, st>>>(amap, umap, p);
  }
  return check_cuda(cudaGetLastError(), "gemm launch");
}

extern "C" size_t q4_gemm_workspace_bytes(int K, int N, int G) {
  if (K <= 0 || N <= 0 || G <= 0) return 0;
  const size_t zp_bytes = ((size_t)G * N * sizeof(__half) + 255) & ~(size_t)255;
  return Q4_GEMM_WS_COUNTER_BYTES + zp_bytes + (size_t)80 * 2 * Q4_GEMM_WS_SLICE_BYTES;
}

extern "C" int q4_gemm_fwd(const void* x, const int32_t* qweight, void* y, const void* scales, const int32_t* qzeros,
                           const int32_t* g_idx, const void* bias, const void* lora_u, const void* lora_b, int lora_r,
                           int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  return gemm_launch(false, x, qweight, y, scales, qzeros, g_idx, bias, lora_u, lora_b, lora_r, M, K, N, G, workspace, workspace_bytes, stream);
}

extern "C" int q4_gemm_fwd_swiglu(const void* x, const int32_t* qweight, void* out, const void* scales, const int32_t* qzeros,
                                  const void* zero_terms, const int32_t* g_idx, const void* bias, int M, int K, int N, int G,
                                  int sequential_groupsize, void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  if (zero_terms && !aligned16(zero_terms)) return fail(Q4_E_ALIGN, "gemm_fwd_swiglu: the zero-term table must be 16-byte aligned");
  return gemm_launch(false, x, qweight, out, scales, qzeros, g_idx, bias, nullptr, nullptr, 0, M, K, N, G, workspace, workspace_bytes, stream,
                     true, zero_terms, nullptr, zero_terms ? sequential_groupsize : 0);
}

extern "C" int q4_gemm_bwd(const void* dy, const int32_t* qweight, void* dx, const void* scales, const int32_t* qzeros,
                           const int32_t* g_idx, const void* lora_v, const void* lora_a, int lora_r,
                           int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  return gemm_launch(true, dy, qweight, dx, scales, qzeros, g_idx, nullptr, lora_v, lora_a, lora_r, M, K, N, G, workspace, workspace_bytes, stream);
}

extern "C" int q4_zero_term_table(const void* scales, const int32_t* qzeros, void* out, int G, int N, q4_stream_t stream) {
  if (!scales || !qzeros || !out) return fail(Q4_E_BADARG, "zero_term_table: null pointer");
  if (G <= 0 || N <= 0 || N % 8) return fail(Q4_E_SHAPE, "zero_term_table: G=%d N=%d (N a multiple of 8)", G, N);
  if (!aligned16(scales) || !aligned16(out)) return fail(Q4_E_ALIGN, "zero_term_table: pointers must be 16-byte aligned");
  if (int e = check_device()) return e;
  const int total8 = G * (N / 8);
  zp_table_kernel<<<(total8 + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const __half*)scales, (const uint32_t*)qzeros, (__half*)out, total8);
  return check_cuda(cudaGetLastError(), "zero_term_table launch");
}

extern "C" int q4_gemm_bwd_table(const void* dy, const int32_t* qweight, void* dx, const void* scales, const int32_t* qzeros,
                                 const void* zero_terms, const int32_t* g_idx, const void* lora_v, const void* lora_a, int lora_r,
                                 int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  if (!zero_terms || !aligned16(zero_terms)) return fail(Q4_E_BADARG, "gemm_bwd_table: needs a 16-byte aligned zero-term table");
  return gemm_launch(true, dy, qweight, dx, scales, qzeros, g_idx, nullptr, lora_v, lora_a, lora_r, M, K, N, G, workspace, workspace_bytes, stream,
                     false, zero_terms);
}

extern "C" int q4_gemm_fwd_table(const void* x, const int32_t* qweight, void* y, const void* scales, const int32_t* qzeros,
                                 const void* zero_terms, const int32_t* g_idx, const void* bias, const void* lora_u, const void* lora_b,
                                 int lora_r, int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  if (!zero_terms || !aligned16(zero_terms)) return fail(Q4_E_BADARG, "gemm_fwd_table: needs a 16-byte aligned zero-term table");
  return gemm_launch(false, x, qweight, y, scales, qzeros, g_idx, bias, lora_u, lora_b, lora_r, M, K, N, G, workspace, workspace_bytes, stream,
                     false, zero_terms);
}

extern "C" int q4_gemm_fwd_residual(const void* x, const int32_t* qweight, void* y, const void* scales, const int32_t* qzeros,
                                    const void* zero_terms, const int32_t* g_idx, const void* bias, const void* residual,
                                    const void* lora_u, const void* lora_b, int lora_r, int M, int K, int N, int G,
                                    int sequential_groupsize, void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  if (zero_terms && !aligned16(zero_terms)) return fail(Q4_E_ALIGN, "gemm_fwd_residual: the zero-term table must be 16-byte aligned");
  return gemm_launch(false, x, qweight, y, scales, qzeros, g_idx, bias, lora_u, lora_b, lora_r, M, K, N, G, workspace, workspace_bytes, stream,
                     false, zero_terms, residual, zero_terms ? sequential_groupsize : 0);
}

extern "C" int q4_gemm_set_variant(int variant) {
  if (variant < 0 || variant > 5)
    return fail(Q4_E_BADARG, "gemm_set_variant: %d is not 0 (choose per shape), 1 (single CTA), 2 (CTA pair, 256-row tiles), 3 (CTA pair, 512-row tiles), "
                "4 (weights in TMEM) or 5 (choose per shape among 1-3)", variant);
  g_gemm_variant = variant;
  return Q4_OK;
}

extern "C" int q4_gemm_set_trace(void* device_buffer) {
  g_gemm_trace = (unsigned long long*)device_buffer;
  return Q4_OK;
}

extern "C" int q4_device_status(unsigned* out) {
  if (!out) return fail(Q4_E_BADARG, "device_status: null pointer");
  return check_cuda(cudaMemcpyFromSymbol(out, g_gemm_status, sizeof(unsigned)), "read device status");
}
