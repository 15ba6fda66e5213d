// The fused dequant-GEMM on CTA pairs (tcgen05 cta_group::2), persistent over output tiles.
// Included by q4_gemm.cu after GemmParams / wait_bar / g_gemm_status are defined.
//
// A pair of CTAs (a cluster of two, on the two SMs of one TPC) computes output tiles of 256 columns
// and 256 or 512 rows: CTA r of the pair holds half of the tile's activation rows and dequantises
// the tile's output columns 128r..128r+127; one tcgen05.mma (M 256 x N 256 x K 16) issued by the even
// CTA multiplies 128 rows of each CTA by all 256 columns and leaves the products in the TMEM of the
// CTA that holds the rows.  Per 16 contraction elements each SM reads 8 KiB of operands for
// 128 x 256 x 16 multiply-adds - half the shared-memory traffic per flop of a single-CTA 128 x 128
// instruction, which is what bounds that form.
//
// The grid is one pair per pair of SMs.  Work is dealt either as whole tiles (pair q takes tiles q,
// q + pairs, ...) or, when that would leave pairs idle in the last round, as equal runs of the
// sequence of all tiles x contraction stages (see WorkItem below).  With 256-row tiles TMEM holds two
// accumulators, so the epilogue of a tile overlaps the MMAs of the next; with 512-row tiles both
// accumulators belong to the tile in flight and every dequantised operand feeds two MMAs.
// Roles (512 threads per CTA):
//   warp 0        TMA producer for this CTA's activation rows; completion bytes of both CTAs are
//                 counted on the even CTA's barrier
//   warp 1        owns TMEM; in the even CTA one elected thread issues the MMAs and the commits
//   warps 2-4, 6-8, 10-11   two groups of four dequantise W for alternate pipeline stages (as in
//                 the single-CTA kernel) and arrive on the even CTA's barrier
//   warps 12-15   epilogue: tcgen05.ld -> (+bias) -> fp16 -> global, one TMEM lane quarter each
// Every wait is bounded; on expiry a status word is set and the kernel runs on without waiting.
#pragma once

namespace q4 {

constexpr int G2_TILE_N = 256;                // output columns per pair (128 dequantised per CTA)
constexpr int G2_HALF_BYTES = 128 * GM_TILE_C * 2;        // 16 KiB: 128 activation rows of one stage
constexpr int G2_B_BYTES = 128 * 64 * 2;                  // 16 KiB: this CTA's columns of the stage
constexpr int G2_MAX_STAGES = 6;
constexpr int G2_THREADS = 512;
constexpr int G2_TMEM_COLS = 512;             // two accumulators of 256 fp32 columns
constexpr int G2_BAR_BYTES = 512;

// Wait of the MMA thread, the pacemaker of the pipeline: single-instruction tests back to back.
__device__ __forceinline__ bool wait_bar_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned* polls = nullptr) {
  if (mbar_test_wait_cluster(bar, parity)) return true;
  const uint32_t lim = *abort_flag ? 4u : 40000000u;
  for (uint32_t i = 0; i < lim; ++i) {
    if (polls) ++*polls;
    if (mbar_test_wait_cluster(bar, parity)) return true;
  }
  *abort_flag = 1;
  atomicExch(&g_gemm_status, Q4_STATUS_WAIT_EXPIRED);
  return false;
}

// Wait of a warp that has nothing else to do for a while (the epilogue between tiles, the TMA
// producer ahead of the MMAs, a dequant warp ahead of the MMAs): sleeps between tests so that its
// polling takes no issue slots from the working warps on the same scheduler.
__device__ __forceinline__ bool wait_bar_idle(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t sleep_ns, unsigned* polls = nullptr) {
  if (mbar_test_wait(bar, parity)) return true;
  const uint32_t lim = *abort_flag ? 4u : 100000000u / sleep_ns;     // about 0.1 s
  for (uint32_t i = 0; i < lim; ++i) {
    if (polls) ++*polls;
    __nanosleep(sleep_ns);
    if (mbar_test_wait(bar, parity)) return true;
  }
  *abort_flag = 1;
  atomicExch(&g_gemm_status, Q4_STATUS_WAIT_EXPIRED);
  return false;
}

// Trace of one launch in nanoseconds of the global timer (slots 100.. of the CTA's 256): where a CTA's time goes.
__device__ __forceinline__ void gm_mark_ns(unsigned long long* tr, int slot) {
  if (tr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    tr[(size_t)blockIdx.x * 256 + slot] = t;
  }
}

// A work item: an output tile, or a run of contraction stages of one.
// SPLIT = false: pair q takes the tiles q, q + pairs, ... whole.
// SPLIT = true ("stream-K"): all tiles x contraction stages, tile by tile, are one sequence that is
// cut into equal runs, one per pair; a run covers the end of one tile, some whole tiles and the
// start of another.  A tile that several pairs contribute to is added up in global memory: every
// contributor writes its fp32 partial sums, the one that arrives last at the tile's counter adds
// them in pair order (the same order whoever is last) and writes the output.
struct WorkItem {
  int tile;      // output tile
  int kb, ke;    // contraction stages [kb, ke)
  bool split;    // partial sum: goes to the workspace instead of the output
  bool lora;     // the low-rank stage follows the contraction stages (the run reaches the end of the tile)
};
struct WorkRange { int first_tile, n_items; unsigned s0, s1; };   // SPLIT: this pair's run [s0, s1) of the stage sequence

template <bool SPLIT>
__device__ __forceinline__ WorkRange work_range(int pair, int n_pairs, int n_tiles, int T) {
  WorkRange r;
  if (!SPLIT) {
    r.first_tile = pair; r.n_items = pair < n_tiles ? (n_tiles - pair + n_pairs - 1) / n_pairs : 0; r.s0 = r.s1 = 0;
  } else {
    const unsigned total = (unsigned)n_tiles * (unsigned)T;        // the host keeps total * pairs below 2^32
    r.s0 = (unsigned)pair * total / (unsigned)n_pairs; r.s1 = ((unsigned)pair + 1u) * total / (unsigned)n_pairs;
    r.first_tile = (int)(r.s0 / (unsigned)T);
    r.n_items = r.s1 > r.s0 ? (int)((r.s1 - 1u) / (unsigned)T) - r.first_tile + 1 : 0;
  }
  return r;
}
template <bool SPLIT>
__device__ __forceinline__ WorkItem work_item(const GemmParams& p, const WorkRange& r, int i, int n_pairs, int T) {
  WorkItem w;
  if (!SPLIT) {
    w.tile = r.first_tile + i * n_pairs; w.kb = 0; w.ke = T; w.split = false; w.lora = p.lora_r > 0;
  } else {
    w.tile = r.first_tile + i;
    const int t0 = w.tile * T;
    w.kb = i == 0 ? (int)r.s0 - t0 : 0;
    w.ke = min(T, (int)r.s1 - t0);
    w.split = w.kb > 0 || w.ke < T;
    w.lora = p.lora_r > 0 && w.ke == T;
  }
  return w;
}
// Pair that owns stage u of the sequence when `total` stages are dealt to `n` pairs as [q total / n, (q + 1) total / n).
__device__ __forceinline__ int stage_owner(long long u, int n, long long total) { return (int)(((u + 1) * n + total - 1) / total) - 1; }

// MH = 1: 256-row tiles (128 rows per CTA) and two TMEM accumulators, so that the epilogue of a tile
// overlaps the MMAs of the next.  MH = 2: 512-row tiles (256 rows per CTA, two MMAs per 16
// contraction elements on the same dequantised operand): half the dequant work per flop, which is
// what bounds the MH = 1 form; both accumulators belong to the one tile in flight.
// SWIGLU (forward only): the layer is a fused [gate | up] projection of 2 I columns and the output is
// half(silu(half(gate))) * half(up), [M, I]: the even CTA of a pair dequantises 128 gate columns, the odd CTA the
// 128 up columns of the same positions, so every accumulator row holds both operands of 128 outputs and the
// product is taken in the epilogue (the roundings are those of the gate_up product followed by the SwiGLU kernel).
template <bool TRANSPOSE, bool SPLIT, int MH, bool SWIGLU = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
q4_gemm2_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap umap, const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);      // 1024-byte aligned, still a shared-space pointer
  unsigned char* stages = smem;
  constexpr int G2_A_BYTES = MH * G2_HALF_BYTES;       // this CTA's activation rows of a stage
  constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
  constexpr int G2_TILE_M = 256 * MH;                  // output rows per pair
  const int S = p.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * G2_STAGE_BYTES);     // even CTA: activation bytes + 4 dequant warps, of both CTAs
  uint64_t* empty = full + 8;                                                   // both CTAs: stage read by the MMAs
  uint64_t* acc_full = empty + 8;                                               // [2] both CTAs: accumulator complete
  uint64_t* acc_empty = acc_full + 2;                                           // [2] even CTA: 4 epilogue warps x 2 CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // forward: [G][128 scales | 128 rn(s*(z+1))], 512 bytes per group
  unsigned char* tab = smem + S * G2_STAGE_BYTES + G2_BAR_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int T = p.n_contract_tiles;
  const int lora_ks = (p.lora_r + 15) >> 4;           // its 16-wide MMA steps
  const int n_out_total = TRANSPOSE ? p.K : p.N;
  const int m_tiles = (p.M + G2_TILE_M - 1) / G2_TILE_M;
  const int n_tiles = m_tiles * (n_out_total / G2_TILE_N);
  const WorkRange wr = work_range<SPLIT>(pair, n_pairs, n_tiles, T);

  if (threadIdx.x == 0) {
    gm_mark_ns(p.trace, 100);
    for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1 + 8); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&amap);
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, G2_TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  if (threadIdx.x == 0) gm_mark_ns(p.trace, 101);

  // Warp w issues on scheduler w % 4.  The MMA warp (1) shares its scheduler with no dequant warp:
  // its short instruction stream is the pacemaker of the whole pipeline and must not queue behind
  // long arithmetic sequences.  Warps 5 and 9 therefore stay idle.
  const int dw = (warp >= 2 && warp <= 11 && warp != 5 && warp != 9) ? warp - 2 - (warp > 5) - (warp > 9) : -1;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's 128 activation rows of every stage ----------------
    if (lane == 0) {
      int st = 0, use = 0;                             // stage and how often it has been used, over all tiles
      unsigned polls = 0;
      const uint32_t full0 = mapa_u32(smem_u32(full), 0);
      for (int item = 0; item < wr.n_items; ++item) {
        const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
        const int m0 = (wi.tile % m_tiles) * G2_TILE_M + 128 * MH * (int)rank;
        const int nst = wi.ke - wi.kb + (wi.lora ? 1 : 0);
        for (int j = 0; j < nst; ++j) {
          const int it = wi.kb + j;
          if (use > 0) wait_bar_idle(&empty[st], (use - 1) & 1, abort_flag, 200, &polls);
          if (rank == 0) mbar_arrive_expect_tx(&full[st], 2 * G2_A_BYTES);
          unsigned char* dst = stages + (size_t)st * G2_STAGE_BYTES;
          if (it < wi.ke) tma_load_2d_pair(dst, &amap, it * GM_TILE_C, m0, full0 + 8 * st);
          else tma_load_2d_pair(dst, &umap, 0, m0, full0 + 8 * st);
          if (++st == S) { st = 0; ++use; }
        }
      }
      if (p.trace) p.trace[(size_t)blockIdx.x * 256 + 240] = polls;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    // The whole warp walks the loop, so that stage counters and descriptors are warp-uniform values (uniform
    // registers, where the tensor-core instructions take their operands from) and one elected lane issues: with a
    // single lane in a divergent branch every operand took a trip through the vector registers, and 4 MMAs + commit
    // cost the issuing thread 850 cycles where the MMAs need 540.
    if (rank == 0) {
      uint32_t leader;
      asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(leader));
      constexpr uint32_t idesc = idesc_f16(256, 256, !TRANSPOSE);
      // descriptors of stage 0; the same descriptors address the same offsets in both CTAs' shared memory.
      // A: K-major, 128-byte rows, 8-row groups 1024 B apart, 16 contraction elements = 32 B.
      // forward  B: MN-major: 64 n contiguous (128 B) per k-row, next 64 n at +8192, 16 k-rows = 2048 B
      // backward B: K-major like A
      const uint64_t ad0 = smem_desc_sw128(smem_u32(stages), 16, 1024);
      const uint64_t bd0 = TRANSPOSE ? smem_desc_sw128(smem_u32(stages) + G2_A_BYTES, 16, 1024)
                                     : smem_desc_sw128(smem_u32(stages) + G2_A_BYTES, 8192, 1024);
      constexpr uint64_t A_STEP = 32 >> 4, B_STEP = (TRANSPOSE ? 32 : 2048) >> 4, ST_STEP = G2_STAGE_BYTES >> 4;
      int st = 0, use = 0, tl = 0;
      unsigned polls = 0;
      uint64_t ad = ad0, bd = bd0;
      for (int item = 0; item < wr.n_items; ++item, ++tl) {
        const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
        const int nst = wi.ke - wi.kb + (wi.lora ? 1 : 0), ncon = wi.ke - wi.kb;
        const int acc = MH == 1 ? (tl & 1) : 0, acc_use = MH == 1 ? (tl >> 1) : tl;
        if (acc_use > 0) wait_bar_cluster(&acc_empty[acc], (acc_use - 1) & 1, abort_flag);
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + acc * 256;
        constexpr uint64_t H_STEP = G2_HALF_BYTES >> 4;   // next 128 activation rows of the stage
        const bool tron = p.trace != nullptr && tl == 1 && lane == 0;
        for (int it = 0; it < nst; ++it) {
          if (tron && it < 12) gm_mark(p.trace, 5 * it);
          wait_bar_cluster(&full[st], use & 1, abort_flag, &polls);
          if (p.trace && lane == 0 && tl == 0 && (it & 7) == 0 && it < 256) gm_mark_ns(p.trace, 110 + (it >> 3));
          if (tron && it < 12) gm_mark(p.trace, 5 * it + 2);
          tc_fence_after();
          if (leader) {
            if (it < ncon) {
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                for (int h = 0; h < MH; ++h)
                  umma_f16_pair(d_tmem + h * 256, ad + ks * A_STEP + h * H_STEP, bd + ks * B_STEP, idesc, (it > 0 || ks > 0) ? 1u : 0u);
            } else {
              for (int ks = 0; ks < lora_ks; ++ks)
#pragma unroll
                for (int h = 0; h < MH; ++h)
                  umma_f16_pair(d_tmem + h * 256, ad + ks * A_STEP + h * H_STEP, bd + ks * B_STEP, idesc, 1u);
            }
            umma_commit_pair(&empty[st]);              // frees the stage in both CTAs
          }
          __syncwarp();
          if (tron && it < 12) gm_mark(p.trace, 5 * it + 4);
          ad += ST_STEP; bd += ST_STEP;
          if (++st == S) { st = 0; ++use; ad = ad0; bd = bd0; }
        }
        if (leader) umma_commit_pair(&acc_full[acc]);
        __syncwarp();
        if (lane == 0 && tl == 0) gm_mark_ns(p.trace, 102);
        if (lane == 0 && item == wr.n_items - 1) gm_mark_ns(p.trace, 103);
      }
      if (p.trace && lane == 0) p.trace[(size_t)blockIdx.x * 256 + 241] = polls;
    }
  } else if (dw >= 0) {
    // ---------------- dequantisers: this CTA's 128 output columns of every stage ----------------
    const int grp = dw >> 2;                                       // takes the stage uses g with g % 2 == grp
    const int tid = ((dw & 3) << 5) | lane;                        // 0..127 within the group
    const int chunk16 = TRANSPOSE ? (tid & 7) : (tid & 15);        // 16-byte chunk (8 columns) within the stage's n-range
    const int r = TRANSPOSE ? (tid >> 3) : (tid >> 4);             // packed row within the stage
    const int N = p.N;
    uint32_t off[8];
    deq_offsets(chunk16 & 7, off);
    const uint32_t full0 = mapa_u32(smem_u32(full), 0);            // the even CTA's full[0]
    int tl = 0, tab_out0 = -1;
    int st = grp, use = 0;                                         // of this group's next stage use (g = grp, grp + 2, ...)
    unsigned polls = 0;
    int gbase = 0;                                                 // stage uses of all earlier items
    for (int item = 0; item < wr.n_items; ++item, ++tl) {
      const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
      const int ncon = wi.ke - wi.kb, nst = ncon + (wi.lora ? 1 : 0);    // stages of this item: j = 0 .. nst-1, contraction stage kb + j
      // first column this CTA dequantises (n forward, k backward)
      const int out0 = SWIGLU ? (wi.tile / m_tiles) * 128 + (int)rank * (p.N >> 1) : (wi.tile / m_tiles) * G2_TILE_N + 128 * (int)rank;
      // packed words of the stage: rows (k0/8 + r), columns ncol0 .. ncol0+7
      auto word_ptr = [&](int it) __attribute__((always_inline)) -> const uint32_t* {
        const int prow = TRANSPOSE ? (out0 >> 3) + r : it * (GM_TILE_C >> 3) + r;
        const int ncol = TRANSPOSE ? it * GM_TILE_C + 8 * chunk16 : out0 + 8 * chunk16;
        return p.qw + (size_t)prow * N + ncol;
      };
      const int j0 = (grp ^ gbase) & 1;                              // this group's first stage of the item
      // Packed words (and, forward, the groups of their 8 k-rows) of one task.  Two sets: the loads of
      // the group's next task are in flight into one while the other is being dequantised.
      struct TaskRegs { uint4 wa, wb; int4 ga, gb; };
      TaskRegs R0, R1;
      int4 tga = make_int4(0, 0, 0, 0), tgb = tga;                   // backward: the task's k-rows are the same in every stage
      // backward, the task's eight rows in one group (always, without act-order) and the zero terms in a table: the
      // task's scales and zero terms are two 16-byte loads, fetched one task ahead with its packed words (they sit in
      // the TaskRegs fields the backward does not use).  Loaded inside the task they put a round trip to L2 in front
      // of every task's arithmetic: the pipeline without any dequant work ran 1.3x faster, with the stores alone 1.25x.
      bool pre_sz = false;
      if (TRANSPOSE) {
        tga = __ldg(reinterpret_cast<const int4*>(p.g_idx + out0 + 8 * r));
        tgb = __ldg(reinterpret_cast<const int4*>(p.g_idx + out0 + 8 * r + 4));
        pre_sz = p.zp_table != nullptr && all_equal8(tga, tgb);
      }
      auto prefetch = [&](int j, TaskRegs& R) __attribute__((always_inline)) {
        if (j >= ncon) return;
        const int it = wi.kb + j;
        R.wa = ldg_stream(word_ptr(it)); R.wb = ldg_stream(word_ptr(it) + 4);
        // The words of the group's task after the next are asked into L2 now: a register prefetch one task
        // ahead covers a hit in L2 but not the trip to HBM that the first reader of a column tile takes
        // (4096 x 4096 at 1024 rows, the same layer again and again: 41.9 -> 37.4 us with this line; 1 % of a
        // LLaMA-7B finetune step, where every layer's words come from HBM).
        if (it + 2 * GM_DEQ_GROUPS < wi.ke) asm volatile("prefetch.global.L2 [%0];" ::"l"(word_ptr(it + 2 * GM_DEQ_GROUPS)));
        if (!TRANSPOSE && p.seq_shift > 0) {         // sequential groups by the caller's word: scales and zero terms ahead, no g_idx
          const size_t at = (size_t)((it * GM_TILE_C + 8 * r) >> p.seq_shift) * N + out0 + 8 * chunk16;
          R.ga = ldg_pinned_int4(p.scales + at);
          R.gb = ldg_pinned_int4(p.zp_table + at);
        } else if (!TRANSPOSE) {
          R.ga = ldg_pinned_int4(p.g_idx + it * GM_TILE_C + 8 * r);
          R.gb = ldg_pinned_int4(p.g_idx + it * GM_TILE_C + 8 * r + 4);
        } else if (pre_sz) {
          const size_t at = (size_t)tga.x * N + it * GM_TILE_C + 8 * chunk16;
          R.ga = ldg_pinned_int4(p.scales + at);
          R.gb = ldg_pinned_int4(p.zp_table + at);
        }
      };
      auto task = [&](int j, const TaskRegs& C) __attribute__((always_inline)) {
        if (st >= S) { st -= S; ++use; }
        unsigned char* bst = stages + (size_t)st * G2_STAGE_BYTES + G2_A_BYTES;
        const int it = wi.kb + j;
        if (j == ncon) {
          // ---- low-rank stage: B operand from lora_w instead of dequantised weights ----
          if (use > 0 && lane == 0) wait_bar_idle(&empty[st], (use - 1) & 1, abort_flag, 100, &polls);
          __syncwarp();
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
          if (lane == 0) mbar_arrive_cluster(full0 + 8 * st);
          st += GM_DEQ_GROUPS;
          return;
        }
        const uint32_t w[8] = {C.wa.x, C.wa.y, C.wa.z, C.wa.w, C.wb.x, C.wb.y, C.wb.z, C.wb.w};
        const bool tr_on = p.trace && tl == 1 && dw == 0 && lane == 0 && j < 40;
        if (tr_on) gm_mark(p.trace, 64 + 3 * (j >> 1));
        if (use > 0 && lane == 0) wait_bar_idle(&empty[st], (use - 1) & 1, abort_flag, 100, &polls);
        __syncwarp();
        if (tr_on) gm_mark(p.trace, 65 + 3 * (j >> 1));
        // forward: panel (chunk16 / 8) of [64 rows][128 B]; backward: one panel of [128 rows][128 B]
        unsigned char* rows8 = bst + (TRANSPOSE ? r * 1024 : (chunk16 >> 3) * 8192 + r * 1024);
        if (TRANSPOSE) {
          const int ncol = it * GM_TILE_C + 8 * chunk16;             // global column of the task
          if (pre_sz) {
            const uint4 sv = make_uint4((uint32_t)C.ga.x, (uint32_t)C.ga.y, (uint32_t)C.ga.z, (uint32_t)C.ga.w);
            const uint4 zv = make_uint4((uint32_t)C.gb.x, (uint32_t)C.gb.y, (uint32_t)C.gb.z, (uint32_t)C.gb.w);
            deq_task_uniform(rows8, off, w, sv, zv);
          } else if (p.zp_table) deq_task_global_zp(rows8, off, w, tga, tgb, p.scales + ncol, p.zp_table + ncol, N);
          else deq_task_global(rows8, off, w, tga, tgb, p.scales + ncol, p.qzeros + (ncol >> 3), N);
        } else if (p.seq_shift > 0) {                // forward, sequential groups: everything the task needs came with its words
          const uint4 sv = make_uint4((uint32_t)C.ga.x, (uint32_t)C.ga.y, (uint32_t)C.ga.z, (uint32_t)C.ga.w);
          const uint4 zv = make_uint4((uint32_t)C.gb.x, (uint32_t)C.gb.y, (uint32_t)C.gb.z, (uint32_t)C.gb.w);
          deq_task_uniform(rows8, off, w, sv, zv);
        } else if (p.zp_table) {                     // forward without shared-memory tables: the caller keeps the zero terms
          const int ncol = out0 + 8 * chunk16;
          deq_task_global_zp(rows8, off, w, C.ga, C.gb, p.scales + ncol, p.zp_table + ncol, N);
        } else {
          deq_task_tables(rows8, off, w, C.ga, C.gb, tab + 16 * chunk16);
        }
        fence_async_smem();                          // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(full0 + 8 * st);
        if (tr_on) gm_mark(p.trace, 66 + 3 * (j >> 1));
        st += GM_DEQ_GROUPS;
      };
      prefetch(j0, R0);                              // in flight while the tables below are built
      if (!TRANSPOSE && !p.zp_table && out0 != tab_out0) {
        // tables for the CTA's 128 columns: scale and rn(s*(z+1)) of every group
        if (tab_out0 >= 0) named_bar_sync(1, GM_DEQ_THREADS * GM_DEQ_GROUPS);      // all readers of the old tables are done
        for (int i = (dw << 5) | lane; i < p.G * 16; i += GM_DEQ_THREADS * GM_DEQ_GROUPS) {
          const int g = i >> 4, c8 = i & 15;
          const uint4 s = __ldg(reinterpret_cast<const uint4*>(p.scales + (size_t)g * N + out0 + 8 * c8));
          const uint32_t zw = __ldg(p.qzeros + (size_t)g * (N >> 3) + ((out0 + 8 * c8) >> 3));
          const uint4 z = zero_terms(s, zw);
          *reinterpret_cast<uint4*>(tab + g * 512 + 16 * c8) = s;
          *reinterpret_cast<uint4*>(tab + g * 512 + 256 + 16 * c8) = z;
        }
        named_bar_sync(1, GM_DEQ_THREADS * GM_DEQ_GROUPS);
        if (tl == 0 && dw == 0 && lane == 0) gm_mark_ns(p.trace, 104);
        tab_out0 = out0;
      }
      for (int j = j0; j < nst; j += 2 * GM_DEQ_GROUPS) {
        prefetch(j + GM_DEQ_GROUPS, R1);
        task(j, R0);
        if (j + GM_DEQ_GROUPS < nst) {
          prefetch(j + 2 * GM_DEQ_GROUPS, R0);
          task(j + GM_DEQ_GROUPS, R1);
        }
      }
      gbase += nst;
    }
    if (p.trace && lane == 0) p.trace[(size_t)blockIdx.x * 256 + 246 + dw] = polls;
  } else if (warp >= 12) {
    // ---------------- epilogue: TMEM -> registers -> (+bias) -> fp16 -> global ----------------
    const int quarter = warp & 3;                                  // TMEM lanes 32*quarter .. +31
    const uint32_t acc_empty0 = mapa_u32(smem_u32(acc_empty), 0);  // the even CTA's acc_empty[0]
    const bool out_aligned32 = (reinterpret_cast<uintptr_t>(p.out) & 31) == 0;   // rows are multiples of 512 bytes apart
    int tl = 0;
    unsigned polls = 0;
    for (int item = 0; item < wr.n_items; ++item, ++tl) {
      const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
      const int acc = MH == 1 ? (tl & 1) : 0, acc_use = MH == 1 ? (tl >> 1) : tl;
      const int col0 = (wi.tile / m_tiles) * (SWIGLU ? 128 : G2_TILE_N);
      const int out_pitch = SWIGLU ? (p.N >> 1) : n_out_total;
      int m = 0;                                                     // output row of this thread, set per accumulator below
      // 32 fp32 sums of row m, columns col0 + 32 cb ..: (+bias) -> fp16 -> global
      auto emit = [&](int cb, const uint32_t (&v)[32]) {
        if (m >= p.M) return;
        __half* dst = p.out + (size_t)m * out_pitch + col0 + cb * 32;
        uint32_t o[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float f0 = __uint_as_float(v[2 * e]), f1 = __uint_as_float(v[2 * e + 1]);
          if (!TRANSPOSE && p.bias) {
            f0 += __half2float(p.bias[col0 + cb * 32 + 2 * e]);
            f1 += __half2float(p.bias[col0 + cb * 32 + 2 * e + 1]);
          }
          o[e] = as_u32(__floats2half2_rn(f0, f1));
        }
        if (!TRANSPOSE && !SWIGLU && p.residual) {         // y = x W + bias + residual: the add of the decoder layer's skip path
          const uint4* rp = reinterpret_cast<const uint4*>(p.residual + (size_t)m * out_pitch + col0 + cb * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 rv = __ldg(rp + q);
            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 a = __half22float2(as_h2(o[4 * q + e])), b = __half22float2(as_h2(rw[e]));
              o[4 * q + e] = as_u32(__floats2half2_rn(a.x + b.x, a.y + b.y));
            }
          }
        }
        if (out_aligned32) {                               // whole 32-byte sectors per store instruction
          asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]),
                       "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
          asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 16), "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]),
                       "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]) : "memory");
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
        }
      };
      if (threadIdx.x == 384 && tl < 8) gm_mark(p.trace, 200 + 3 * tl);
      if (lane == 0) wait_bar_idle(&acc_full[acc], acc_use & 1, abort_flag, 250, &polls);
      __syncwarp();
      tc_fence_after();
      if (threadIdx.x == 384 && tl < 8) gm_mark(p.trace, 201 + 3 * tl);
      if (threadIdx.x == 384 && item == wr.n_items - 1) gm_mark_ns(p.trace, 105);
      // Partial sums of a run: this warp's 32 rows x 256 columns of accumulator h as
      // [cb][j][lane][4 floats], so that every 16-byte access of the warp is one contiguous 512 bytes.
      // Blocks are indexed [contributing pair][CTA of the pair][accumulator][lane quarter].
      // The pair whose run STARTS a shared tile adds the tile up: that piece is the last item of its
      // run, so the other contributors (for whom the tile comes earlier in their runs) have as a rule
      // long published their sums; it adds them to its own accumulator in pair order.
      const size_t part_floats = 8 * 8 * 32 * 4;
      auto part_of = [&](int cpair, int h) -> float* {
        return p.ws_partials + ((((size_t)cpair * 2 + rank) * MH + h) * 4 + quarter) * part_floats;
      };
      const bool shared_tile = SPLIT && wi.split;
      const bool reducer = shared_tile && wi.kb == 0;
      int c_first = 0, c_last = 0;
      unsigned* cnt = nullptr;
      if (shared_tile) {
        const long long total = (long long)n_tiles * T;
        c_first = stage_owner((long long)wi.tile * T, n_pairs, total);
        c_last = stage_owner((long long)wi.tile * T + T - 1, n_pairs, total);
        cnt = p.ws_counters + ((size_t)c_first * 2 + rank) * 4 + quarter;     // a pair starts at most one shared tile
      }
      if (reducer) {
        if (lane == 0) {
          const unsigned want = (unsigned)(c_last - c_first);
          bool ok = false;
          const uint32_t lim = *abort_flag ? 4u : 500000u;                    // x 200 ns
          for (uint32_t i = 0; i < lim && !ok; ++i) {
            unsigned have;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(have) : "l"(cnt) : "memory");
            ok = have >= want;
            if (!ok) __nanosleep(200);
          }
          if (!ok) { *abort_flag = 1; atomicExch(&g_gemm_status, Q4_STATUS_WAIT_EXPIRED); }
        }
        __syncwarp();
        __threadfence();
      }
#pragma unroll 1
      for (int h = 0; h < MH; ++h) {
        m = (wi.tile % m_tiles) * G2_TILE_M + 128 * MH * (int)rank + 128 * h + 32 * quarter + lane;
        float* part = shared_tile && !reducer ? part_of(pair, h) : nullptr;
        // what happens to 32 sums of this thread's row: output, partial sums, or output of the sum over all contributors
        auto consume = [&](int cb, uint32_t (&v)[32]) {
          if (!shared_tile) {
            emit(cb, v);
          } else if (!reducer) {
            if (m < p.M) {                                 // rows beyond M are padding: nobody reads their sums
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(part + ((cb * 8 + j) * 32 + lane) * 4) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
          }
        };
        const uint32_t tsrc = tmem_acc + ((uint32_t)(32 * quarter) << 16) + (acc + h) * 256;
        if constexpr (SWIGLU) {
          // accumulator columns 32 cb .. (gate) and 128 + 32 cb .. (up) of this thread's row together
#pragma unroll 1
          for (int cb = 0; cb < 4; ++cb) {
            uint32_t gv[32], uv[32];
            __syncwarp();                                  // the lanes of rows past M skipped the stores: whole again for the aligned load
            tmem_ld32(tsrc + cb * 32, gv);
            tmem_ld32(tsrc + 128 + cb * 32, uv);
            tmem_ld_wait();
            if (shared_tile && !reducer) {
              if (m < p.M) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  *reinterpret_cast<uint4*>(part + ((cb * 8 + j) * 32 + lane) * 4) = make_uint4(gv[4 * j], gv[4 * j + 1], gv[4 * j + 2], gv[4 * j + 3]);
                  *reinterpret_cast<uint4*>(part + (((cb + 4) * 8 + j) * 32 + lane) * 4) = make_uint4(uv[4 * j], uv[4 * j + 1], uv[4 * j + 2], uv[4 * j + 3]);
                }
              }
              continue;
            }
            if (reducer) {
              for (int cc = c_first + 1; cc <= c_last; ++cc) {
                const float* s2 = part_of(cc, h);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 a = __ldcg(reinterpret_cast<const float4*>(s2 + ((cb * 8 + j) * 32 + lane) * 4));
                  const float4 b = __ldcg(reinterpret_cast<const float4*>(s2 + (((cb + 4) * 8 + j) * 32 + lane) * 4));
                  gv[4 * j] = __float_as_uint(__uint_as_float(gv[4 * j]) + a.x); gv[4 * j + 1] = __float_as_uint(__uint_as_float(gv[4 * j + 1]) + a.y);
                  gv[4 * j + 2] = __float_as_uint(__uint_as_float(gv[4 * j + 2]) + a.z); gv[4 * j + 3] = __float_as_uint(__uint_as_float(gv[4 * j + 3]) + a.w);
                  uv[4 * j] = __float_as_uint(__uint_as_float(uv[4 * j]) + b.x); uv[4 * j + 1] = __float_as_uint(__uint_as_float(uv[4 * j + 1]) + b.y);
                  uv[4 * j + 2] = __float_as_uint(__uint_as_float(uv[4 * j + 2]) + b.z); uv[4 * j + 3] = __float_as_uint(__uint_as_float(uv[4 * j + 3]) + b.w);
                }
              }
            }
            if (m < p.M) {
              __half* dst = p.out + (size_t)m * out_pitch + col0 + cb * 32;
              uint32_t o[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                float g0 = __uint_as_float(gv[2 * e]), g1 = __uint_as_float(gv[2 * e + 1]);
                float u0 = __uint_as_float(uv[2 * e]), u1 = __uint_as_float(uv[2 * e + 1]);
                if (p.bias) {
                  g0 += __half2float(p.bias[col0 + cb * 32 + 2 * e]); g1 += __half2float(p.bias[col0 + cb * 32 + 2 * e + 1]);
                  u0 += __half2float(p.bias[out_pitch + col0 + cb * 32 + 2 * e]); u1 += __half2float(p.bias[out_pitch + col0 + cb * 32 + 2 * e + 1]);
                }
                const float2 gf = __half22float2(__floats2half2_rn(g0, g1));      // the gate as the unfused product would have stored it
                o[e] = as_u32(__hmul2(__floats2half2_rn(silu_f(gf.x), silu_f(gf.y)), __floats2half2_rn(u0, u1)));
              }
              if (out_aligned32) {
                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]),
                             "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 16), "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]),
                             "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]) : "memory");
              } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
              }
            }
          }
        } else if (!reducer) {                             // (warp-uniform: rows past M of a shared tile add whatever the
                                                           // workspace holds and store nothing)
          // two register buffers: the TMEM load of the next 32 columns is in flight while these are consumed
          // (the lanes of rows past M leave `consume` early: __syncwarp makes the warp whole again before every
          // warp-wide TMEM instruction)
          uint32_t va[32], vb[32];
          __syncwarp();
          tmem_ld32(tsrc, va);
#pragma unroll 1
          for (int cb = 0; cb < G2_TILE_N / 32; cb += 2) {
            tmem_ld_wait();
            tmem_ld32(tsrc + (cb + 1) * 32, vb);
            consume(cb, va);
            __syncwarp();
            tmem_ld_wait();
            if (cb + 2 < G2_TILE_N / 32) tmem_ld32(tsrc + (cb + 2) * 32, va);
            consume(cb + 1, vb);
            __syncwarp();
          }
        } else {
          // adding up a shared tile: what takes long is the first other contributor's sums coming from L2, so
          // the loads of the next block of 32 columns are issued before this block is converted and stored;
          // further contributors (rare) are read on the spot
          const float* src = part_of(c_first + 1, h);
          float4 t[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] = __ldcg(reinterpret_cast<const float4*>(src + (j * 32 + lane) * 4));
#pragma unroll 1
          for (int cb = 0; cb < G2_TILE_N / 32; ++cb) {
            uint32_t v[32];
            __syncwarp();
            tmem_ld32(tsrc + cb * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + t[j].x);
              v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + t[j].y);
              v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + t[j].z);
              v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + t[j].w);
            }
            if (cb + 1 < G2_TILE_N / 32) {
#pragma unroll
              for (int j = 0; j < 8; ++j) t[j] = __ldcg(reinterpret_cast<const float4*>(src + (((cb + 1) * 8 + j) * 32 + lane) * 4));
            }
            for (int cc = c_first + 2; cc <= c_last; ++cc) {
              const float* s2 = part_of(cc, h);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 u = __ldcg(reinterpret_cast<const float4*>(s2 + ((cb * 8 + j) * 32 + lane) * 4));
                v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + u.x);
                v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + u.y);
                v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + u.z);
                v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + u.w);
              }
            }
            emit(cb, v);
          }
        }
      }
      // this warp has read its part of the accumulator(s): the even CTA may overwrite them
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8 * acc);
      if (shared_tile && !reducer) {                       // publish: sums, then the count
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(cnt, 1u);
      }
      if (reducer && lane == 0) *cnt = 0;                  // every contributor has been counted: ready for the next launch
      if (threadIdx.x == 384 && tl < 8) gm_mark(p.trace, 202 + 3 * tl);
    }
    if (p.trace && lane == 0) p.trace[(size_t)blockIdx.x * 256 + 242 + (warp & 3)] = polls;
  }
  // neither CTA may leave (or free TMEM) while its peer can still signal its barriers or read its tiles
  if (threadIdx.x == 384) gm_mark_ns(p.trace, 106);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (threadIdx.x == 0) gm_mark_ns(p.trace, 107);
  if (warp == 1) tmem_dealloc_pair(tmem_acc, G2_TMEM_COLS);
}

static size_t gemm2_smem_bytes(bool transpose, int G, int stages, int mh) {
  return 1024 + (size_t)stages * (mh * G2_HALF_BYTES + G2_B_BYTES) + G2_BAR_BYTES + (transpose ? 0 : (size_t)2 * G * 128 * sizeof(__half));
}

// Pipeline depth the pair kernel gets for this layer (0 = its tables do not leave room for three stages).
static int gemm2_stages(bool transpose, int G, int mh) {
  int stages = G2_MAX_STAGES;
  while (stages > 2 && gemm2_smem_bytes(transpose, G, stages, mh) > 227 * 1024) --stages;
  return stages >= 3 ? stages : 0;
}

}  // namespace q4
