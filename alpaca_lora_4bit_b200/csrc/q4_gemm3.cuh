// The fused dequant-GEMM forward with the dequantised weights in TENSOR MEMORY (tcgen05.mma with its A operand
// in TMEM), for layers whose groups are sequential by the caller's word.  Included by q4_gemm.cu after q4_gemm2.cuh.
//
// The pair kernel of q4_gemm2.cuh keeps both operands in shared memory: a dequant task there is eight swizzled
// 16-byte stores behind scale and zero-term vectors of eight columns, a proxy fence and a barrier, and per 64
// contraction elements an SM takes 16 KiB of dequant stores on top of 16 KiB of TMA writes and 32 KiB of tensor-core
// reads.  Here the product is transposed,
// y^T = W^T x^T: the weights are the A operand (M side: 256 output columns per pair, 128 per CTA = one TMEM lane
// each), the activations the B operand (N side: 256 rows of x per tile, 128 per CTA, K-major by TMA exactly as
// before).  A dequant thread owns one output column: the eight packed words of its column and a stage are eight
// coalesced 4-byte loads, one word is eight consecutive k of that column = four half2 in contraction order, scale
// and zero term are scalars of the thread, and the stage's 64 halves leave as one `tcgen05.st` of 32 columns.
// Nothing of W touches shared memory; an SM moves 16 KiB of TMA writes and 16 KiB of operand reads per stage.
//
// TMEM (512 columns): accumulator [128 lanes = output columns][256 columns = rows of x] fp32, and eight operand
// stages of 32 columns (lane = output column, column c of a stage = contraction elements 2c, 2c+1 as a half2).
// Roles (640 threads per CTA): warp 0 TMA producer of this CTA's 128 activation rows; warp 1 owns TMEM, its elected
// lane in the even CTA issues the MMAs; warps 4-15 dequantise (warp & 3 = its TMEM lane quarter; three groups of
// four warps take every third stage use: a task is a chain of loads, arithmetic, the wait for the slot, the TMEM
// store and its completion, about 1500 cycles where the MMAs of a stage take 540, so three tasks have to be in
// flight); warps 16-19 epilogue.  Whole tiles per pair round after round, or (SPLIT) equal runs of tiles x stages.
// The accumulator's lanes are output columns, so a thread of the epilogue holds 32 rows of one column: a warp
// first moves its 32 columns x 256 rows into shared memory as fp16 (and hands the accumulator back: the MMAs of the
// pair's next item start while the stores run), then stores rows of 64 bytes, four lanes each.
// Every wait is bounded as in the pair kernel.
#pragma once

namespace q4 {

constexpr int G3_STAGES = 8;                  // operand stages in TMEM = activation stages in shared memory
static_assert(G3_STAGES == 8, "a stage use u lies in slot u & 7, use u >> 3");
constexpr int G3_X_BYTES = 128 * GM_TILE_C * 2;           // 16 KiB: this CTA's 128 activation rows of a stage
constexpr int G3_TMEM_A0 = 256;               // first TMEM column of the operand stages
constexpr int G3_BAR_BYTES = 512;
constexpr int G3_GROUPS = 3;                  // dequant groups of four warps
constexpr int G3_THREADS = 32 * (4 + 4 * G3_GROUPS + 4);
constexpr int G3_TURN_BYTES = 4 * 256 * 64;    // per epilogue warp its 32 columns of all 256 rows of a tile, fp16

__device__ __forceinline__ void umma_f16_pair_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp writes lane (lane base + i).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
        "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
        "r"(v[30]), "r"(v[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t ldg_pinned_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_pinned_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

// One packed word = eight consecutive contraction elements of one output column -> four half2 in order.
// Byte j of the word holds levels 2j (low nibble) and 2j+1 (high nibble): the byte is copied to bytes 0 and 2,
// the low nibble becomes the mantissa of 1024 + q, the high nibble stays in place as the mantissa of 64 + q
// (exponent 0x5400, ulp 1/16), and one fused multiply-add with (-1024 s, -64 s) leaves rn(s q) in both halves.
template <bool FOLD>
__device__ __forceinline__ void deq_word_k(uint32_t w, uint32_t s2, uint32_t c2, uint32_t z2, uint32_t* o) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t u = prmt(w, w, j | (j << 8));
    const uint32_t v = and_or(u, 0x00F0000Fu, 0x54006400u);
    if (FOLD) o[j] = as_u32(__hsub2_rn(__hfma2(as_h2(v), as_h2(s2), as_h2(c2)), as_h2(z2)));
    else o[j] = as_u32(__hsub2_rn(__hmul2_rn(as_h2(s2), __hsub2(as_h2(v), as_h2(0x54006400u))), as_h2(z2)));
  }
}

// SPLIT as in the pair kernel: whole tiles per pair, or equal runs of the sequence of all tiles x stages with the
// partial sums of a shared tile meeting in the workspace (added in pair order by the pair whose run starts the tile).
template <bool SPLIT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G3_THREADS, 1)
q4_gemm3_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap umap, const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* stages = smem;
  constexpr int S = G3_STAGES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * G3_X_BYTES);          // even CTA: activation bytes + 4 dequant warps, of both CTAs
  uint64_t* empty = full + 8;                                                   // both CTAs: stage read by the MMAs
  uint64_t* acc_full = empty + 8;                                               // both CTAs: accumulator complete
  uint64_t* acc_empty = acc_full + 1;                                           // even CTA: 4 epilogue warps x 2 CTAs
  uint64_t* last_full = acc_empty + 1;                                          // both CTAs: the pair's last accumulator complete (one use)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(last_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned char* turn = smem + S * G3_X_BYTES + G3_BAR_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int T = p.n_contract_tiles;
  const int lora_ks = (p.lora_r + 15) >> 4;
  const int N = p.N;
  const int m_tiles = (p.M + 255) / 256;
  const int n_tiles = m_tiles * (N / G2_TILE_N);
  const WorkRange wr = work_range<SPLIT>(pair, n_pairs, n_tiles, T);
  const int n_items = wr.n_items;

  // A dequant warp asks for the words of its first task before the set-up below (barriers, TMEM, the cluster's
  // meeting: about a microsecond): the loads depend on none of it.
  struct TaskRegs { uint32_t w[8]; uint32_t s, z; };
  const bool is_deq = warp >= 4 && warp < 4 + 4 * G3_GROUPS;
  auto column_of = [&](int tile) { return (tile / m_tiles) * G2_TILE_N + 128 * (int)rank + 32 * (warp & 3) + lane; };
  auto prefetch = [&](int n, int j, TaskRegs& R) __attribute__((always_inline)) {
    if (j >= T) return;
    const uint32_t* wcol = p.qw + n;
    const uint32_t* src = wcol + (size_t)(j * (GM_TILE_C >> 3)) * N;
#pragma unroll
    for (int i = 0; i < 8; ++i) R.w[i] = ldg_pinned_u32(src + (size_t)i * N);
    const size_t at = (size_t)((j * GM_TILE_C) >> p.seq_shift) * N + n;
    R.s = ldg_pinned_u16(p.scales + at);
    R.z = ldg_pinned_u16(p.zp_table + at);
    // the words of the group's task after the next, asked into L2 (eight rows of 128 bytes per warp)
    if (j + 2 * G3_GROUPS < T && lane < 8)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(wcol - lane + (size_t)((j + 2 * G3_GROUPS) * (GM_TILE_C >> 3) + lane) * N));
  };
  TaskRegs R0, R1;
  if (is_deq && n_items > 0) {
    const WorkItem w0 = work_item<SPLIT>(p, wr, 0, n_pairs, T);
    const int n = column_of(w0.tile), j = w0.kb + ((warp - 4) >> 2);
    if (j < w0.ke) prefetch(n, j, R0);
  }

  if (threadIdx.x == 0) {
    gm_mark_ns(p.trace, 100);
    for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1 + 8); mbar_init(&empty[i], 1); }
    mbar_init(acc_full, 1); mbar_init(acc_empty, 8); mbar_init(last_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&amap);
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, G2_TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) gm_mark_ns(p.trace, 101);

  // One block of 32 rows of a warp's 32 output columns: (+bias) -> fp16 -> shared memory, one half per row and lane.
  auto block_to_smem = [&](unsigned char* buf, const uint32_t (&v)[32], float bv) __attribute__((always_inline)) {
#pragma unroll
    for (int t = 0; t < 32; ++t)
      *reinterpret_cast<__half*>(buf + t * 64 + lane * 2) = __float2half_rn(__uint_as_float(v[t]) + bv);
  };
  // ... and from there to global memory: rows of 64 bytes, four lanes each, with the skip-path add
  auto block_to_global = [&](const unsigned char* buf, int m0, int n0) __attribute__((always_inline)) {
    const int rr = lane >> 2, cc = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = rr + 8 * i, m = m0 + r;
      uint4 o = *reinterpret_cast<const uint4*>(buf + r * 64 + cc * 16);
      if (m < p.M) {
        const size_t at = (size_t)m * N + n0 + 8 * cc;
        if (p.residual) {                                          // rounded first, as the separate add of the decoder layer would see it
          const uint4 rv = __ldg(reinterpret_cast<const uint4*>(p.residual + at));
          uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
          const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a = __half22float2(as_h2(ov[e])), b = __half22float2(as_h2(rw[e]));
            ov[e] = as_u32(__floats2half2_rn(a.x + b.x, a.y + b.y));
          }
        }
        *reinterpret_cast<uint4*>(p.out + at) = o;
      }
    }
  };
  // The pair's last item, when it is a whole tile: nothing follows it, so the dequant warps (three per TMEM lane
  // quarter) share its epilogue with the epilogue warp of their quarter, blocks of 32 rows dealt round robin.
  const WorkItem w_last = work_item<SPLIT>(p, wr, n_items > 0 ? n_items - 1 : 0, n_pairs, T);
  const bool share_last = n_items > 0 && !(SPLIT && w_last.split);

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's 128 rows of x (or of lora_u) of every stage ----------------
    if (lane == 0) {
      int st = 0, use = 0;
      const uint32_t full0 = mapa_u32(smem_u32(full), 0);
      for (int item = 0; item < n_items; ++item) {
        const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
        const int m0 = (wi.tile % m_tiles) * 256 + 128 * (int)rank;
        const int nst = wi.ke - wi.kb + (wi.lora ? 1 : 0);
        for (int j = 0; j < nst; ++j) {
          const int it = wi.kb + j;
          if (use > 0) wait_bar_idle(&empty[st], (use - 1) & 1, abort_flag, 40);
          if (rank == 0) mbar_arrive_expect_tx(&full[st], 2 * G3_X_BYTES);
          unsigned char* dst = stages + (size_t)st * G3_X_BYTES;
          if (it < wi.ke) tma_load_2d_pair(dst, &amap, it * GM_TILE_C, m0, full0 + 8 * st);
          else tma_load_2d_pair(dst, &umap, 0, m0, full0 + 8 * st);
          if (++st == S) { st = 0; ++use; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    // The whole warp walks the loop, so that stage counters, descriptors and TMEM addresses are warp-uniform values
    // (uniform registers, which the tensor-core instructions take their operands from); one elected lane issues.
    if (rank == 0) {
      uint32_t leader;
      asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(leader));
      constexpr uint32_t idesc = idesc_f16(256, 256, false);
      // B: this CTA's 128 rows of x, K-major, 128-byte rows, 8-row groups 1024 B apart, 16 contraction elements = 32 B
      const uint64_t bd0 = smem_desc_sw128(smem_u32(stages), 16, 1024);
      constexpr uint64_t B_STEP = 32 >> 4, ST_STEP = G3_X_BYTES >> 4;
      int st = 0, use = 0;
      uint64_t bd = bd0;
      for (int item = 0; item < n_items; ++item) {
        const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
        const int ncon = wi.ke - wi.kb, nst = ncon + (wi.lora ? 1 : 0);
        if (item > 0) wait_bar_cluster(acc_empty, (item - 1) & 1, abort_flag);
        tc_fence_after();
        for (int it = 0; it < nst; ++it) {
          wait_bar_cluster(&full[st], use & 1, abort_flag);
          if (p.trace && lane == 0 && item == 0 && (it & 7) == 0 && it < 64) gm_mark_ns(p.trace, 110 + (it >> 3));
          tc_fence_after();
          const uint32_t a_tmem = tmem_base + G3_TMEM_A0 + 32 * st;
          const int nks = it < ncon ? 4 : lora_ks;
          if (leader) {
            for (int ks = 0; ks < nks; ++ks)
              umma_f16_pair_ts(tmem_base, a_tmem + 8 * ks, bd + ks * B_STEP, idesc, (it > 0 || ks > 0) ? 1u : 0u);
            umma_commit_pair(&empty[st]);
          }
          __syncwarp();
          bd += ST_STEP;
          if (++st == S) { st = 0; ++use; bd = bd0; }
        }
        if (leader) { umma_commit_pair(acc_full); if (item == n_items - 1) umma_commit_pair(last_full); }
        __syncwarp();
        if (lane == 0 && item == 0) gm_mark_ns(p.trace, 102);
        if (lane == 0 && item == n_items - 1) gm_mark_ns(p.trace, 103);
      }
    }
  } else if (warp >= 4 && warp < 4 + 4 * G3_GROUPS) {
    // ---------------- dequantisers: one output column per thread, 64 contraction elements per task ----------------
    const int grp = (warp - 4) >> 2;                               // takes the stage uses u with u % G3_GROUPS == grp
    const int quarter = warp & 3;
    const uint32_t full0 = mapa_u32(smem_u32(full), 0);
    const uint32_t tdst0 = tmem_base + ((uint32_t)(32 * quarter) << 16) + G3_TMEM_A0;
    int gbase = 0;                                                 // stage uses of all earlier tiles
    for (int item = 0; item < n_items; ++item) {
      const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
      const int n = column_of(wi.tile);
      const int ncon = wi.ke - wi.kb, nst = ncon + (wi.lora ? 1 : 0);       // stages of this item: j = 0 .. nst-1, contraction stage kb + j
      auto task = [&](int j, const TaskRegs& C) __attribute__((always_inline)) {
        const int u = gbase + j, st = u & (S - 1), use = u >> 3;
        uint32_t o[32];
        if (j == ncon) {
          // low-rank stage: lane = column n holds lora_B[n][0..r), zero beyond
          const __half* src = p.lora_w + (size_t)n * p.lora_r;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const __half lo = 2 * c < p.lora_r ? src[2 * c] : __float2half(0.f);
            const __half hi = 2 * c + 1 < p.lora_r ? src[2 * c + 1] : __float2half(0.f);
            o[c] = as_u32(__halves2half2(lo, hi));
          }
        } else {
          const uint32_t s2 = prmt(C.s, C.s, 0x1010), z2 = prmt(C.z, C.z, 0x1010);
          if ((C.s & 0x4000u) == 0) {                    // |s| < 2: 1024 s is exact
            const uint32_t c2 = as_u32(__hmul2_rn(as_h2(s2), as_h2(0xD400E400u) /* (-1024, -64) */));
#pragma unroll
            for (int i = 0; i < 8; ++i) deq_word_k<true>(C.w[i], s2, c2, z2, o + 4 * i);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) deq_word_k<false>(C.w[i], s2, 0u, z2, o + 4 * i);
          }
        }
        if (use > 0 && lane == 0) wait_bar_idle(&empty[st], (use - 1) & 1, abort_flag, 40);
        __syncwarp();
        tc_fence_after();
        tmem_st32(tdst0 + 32 * st, o);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(full0 + 8 * st);
      };
      int j = (grp + G3_GROUPS - gbase % G3_GROUPS) % G3_GROUPS;   // this group's first stage of the tile
      auto ask = [&](int jj, TaskRegs& R) __attribute__((always_inline)) { if (jj < ncon) prefetch(n, wi.kb + jj, R); };
      if (item > 0) ask(j, R0);                                    // (the first item's came before the set-up)
      while (j < nst) {
        ask(j + G3_GROUPS, R1);
        task(j, R0);
        j += G3_GROUPS;
        if (j >= nst) break;
        ask(j + G3_GROUPS, R0);
        task(j, R1);
        j += G3_GROUPS;
      }
      gbase += nst;
    }
    if (share_last) {
      const int n0 = (w_last.tile / m_tiles) * G2_TILE_N + 128 * (int)rank + 32 * quarter;
      const int m_base = (w_last.tile % m_tiles) * 256;
      const int nb = (min(256, p.M - m_base) + 31) >> 5;
      const float bv = p.bias ? __half2float(p.bias[n0 + lane]) : 0.f;
      // the quarter's shared-memory rows are free once its epilogue warp has stored the item before (a meeting of
      // the quarter's four warps: named barrier 1 + quarter)
      named_bar_sync(1 + quarter, 128);
      if (lane == 0) wait_bar_idle(last_full, 0, abort_flag, 100);
      __syncwarp();
      tc_fence_after();
      unsigned char* mine = turn + quarter * 16384;
#pragma unroll 1
      for (int cb = grp; cb < nb; cb += G3_GROUPS + 1) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(32 * quarter) << 16) + cb * 32, v);
        tmem_ld_wait();
        block_to_smem(mine + cb * 2048, v, bv);
        __syncwarp();
        block_to_global(mine + cb * 2048, m_base + cb * 32, n0);
      }
    }
  } else if (warp >= 4 + 4 * G3_GROUPS) {
    // ---------------- epilogue: TMEM -> registers -> (+bias) -> fp16 -> turned over in shared memory -> (+residual) -> global ----------------
    const int quarter = warp & 3;
    const uint32_t acc_empty0 = mapa_u32(smem_u32(acc_empty), 0);
    unsigned char* mine = turn + quarter * 16384;                  // [256 rows][32 columns] fp16
    for (int item = 0; item < n_items; ++item) {
      const WorkItem wi = work_item<SPLIT>(p, wr, item, n_pairs, T);
      const int n0 = (wi.tile / m_tiles) * G2_TILE_N + 128 * (int)rank + 32 * quarter;     // this warp's 32 output columns
      const int m_base = (wi.tile % m_tiles) * 256;
      const int rows = min(256, p.M - m_base);                     // rows of x the tile really has
      const float bv = p.bias ? __half2float(p.bias[n0 + lane]) : 0.f;
      if (share_last && item == n_items - 1) named_bar_sync(1 + quarter, 128);     // the helpers may use this quarter's rows from here
      if (lane == 0) wait_bar_idle(acc_full, item & 1, abort_flag, 100);
      __syncwarp();
      tc_fence_after();
      if (lane == 0 && item == n_items - 1) gm_mark_ns(p.trace, 105);
      const uint32_t tsrc = tmem_base + ((uint32_t)(32 * quarter) << 16);
      const int nb = (rows + 31) >> 5;                             // blocks of 32 rows that hold anything
      const bool shared_out = share_last && item == n_items - 1;   // the dequant warps take the blocks cb % 4 = 0, 1, 2
      const int cb0 = shared_out ? G3_GROUPS : 0, cbs = shared_out ? G3_GROUPS + 1 : 1;
      // Partial sums of a run: this warp's 32 columns x 256 rows as [block][j][lane][4 floats] (512 contiguous bytes
      // per 16-byte access of the warp), indexed [contributing pair][CTA of the pair][lane quarter].
      const size_t part_floats = 8 * 8 * 32 * 4;
      auto part_of = [&](int cpair) -> float* { return p.ws_partials + (((size_t)cpair * 2 + rank) * 4 + quarter) * part_floats; };
      const bool shared_tile = SPLIT && wi.split;
      const bool reducer = shared_tile && wi.kb == 0;
      int c_first = 0, c_last = 0;
      unsigned* cnt = nullptr;
      if (shared_tile) {
        const long long total = (long long)n_tiles * T;
        c_first = stage_owner((long long)wi.tile * T, n_pairs, total);
        c_last = stage_owner((long long)wi.tile * T + T - 1, n_pairs, total);
        cnt = p.ws_counters + ((size_t)c_first * 2 + rank) * 4 + quarter;
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
      for (int cb = cb0; cb < nb; cb += cbs) {
        uint32_t v[32];
        tmem_ld32(tsrc + cb * 32, v);
        tmem_ld_wait();
        if (shared_tile && !reducer) {
          float* part = part_of(pair);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(part + ((cb * 8 + q) * 32 + lane) * 4) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          continue;
        }
        if (reducer) {
          for (int c2 = c_first + 1; c2 <= c_last; ++c2) {
            const float* src = part_of(c2);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 a = __ldcg(reinterpret_cast<const float4*>(src + ((cb * 8 + q) * 32 + lane) * 4));
              v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + a.x); v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + a.y);
              v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + a.z); v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + a.w);
            }
          }
        }
        block_to_smem(mine + cb * 2048, v, bv);
      }
      // this warp has read its part of the accumulator: the even CTA may start the next item
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0);
      if (!(shared_tile && !reducer)) {
#pragma unroll 1
        for (int cb = cb0; cb < nb; cb += cbs) block_to_global(mine + cb * 2048, m_base + cb * 32, n0);
        __syncwarp();                                      // the rows are read before the next item overwrites them
      }
      if (shared_tile && !reducer) {                       // publish: sums, then the count
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(cnt, 1u);
      }
      if (reducer && lane == 0) *cnt = 0;                  // every contributor has been counted: ready for the next launch
    }
  }
  if (threadIdx.x == G3_THREADS - 128) gm_mark_ns(p.trace, 106);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (threadIdx.x == 0) gm_mark_ns(p.trace, 107);
  if (warp == 1) tmem_dealloc_pair(tmem_base, G2_TMEM_COLS);
}

static size_t gemm3_smem_bytes() { return 1024 + (size_t)G3_STAGES * G3_X_BYTES + G3_BAR_BYTES + G3_TURN_BYTES; }

}  // namespace q4
