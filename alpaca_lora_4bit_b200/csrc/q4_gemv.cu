// Decode product  y[M,N] (+)= x[M,K] * W  for 1 <= M <= 16 straight from the packed int4 layer.
//
// Per weight 0.5 B of qweight plus 1/64 B of scales and 1/256 B of zero points cross HBM at groupsize
// 128; x and y are noise.  Five kernels share the file; q4_gemv at its end picks one per call:
//   * gemv_ws_kernel     one row, groups of 128, K in whole 256-row units: warp-specialised (a copy-issuing
//                        warp, consumer warps, a helper for the exchange between CTAs), int8 tensor-core
//                        MMAs on the packed words split into bytes, x as 16-bit block fixed point.
//   * gemv_rows_kernel   2..16 rows on the same layers, one pass over the weights: the same int8 MMAs, x
//                        converted to block fixed point once per call by x_convert_kernel (an 8-row and a
//                        16-row form).
//   * gemv_fast_kernel   1..8 rows (9..16: two launches) where the two above do not apply - groups of a
//                        multiple of 256 rows, the first layer format, layers with few column tiles: every
//                        warp streams its own 4 KiB units with TMA, fp16 MMAs with the exponent trick, x
//                        re-laid per unit or once per CTA.
//   * gemv_stream_kernel every other group size with sequential groups: the same streams, group test per step.
//   * gemv_act_kernel    act-order (the group of every row from g_idx): scale and zero point per element
//                        from shared-memory tables.
// Common to all: the matrix is cut into units of 32 packed rows x 32 columns (4 KiB = 256 k-rows of one
// 32-column tile) that arrive by TMA on mbarriers; W is the A operand of mma.sync (rows = output columns),
// x the B operand (columns = batch rows); sums are kept in fp32 (or exact integers) and added in a fixed
// order, so results are reproducible; launches carry the programmatic-dependent-launch attribute and wait
// for the earlier kernel only before they first touch x, y or the workspace (weights never depend on an
// earlier kernel); every wait on a barrier or a flag is bounded - on expiry the kernel records a status word
// in the workspace (q4_gemv_status), stops waiting and runs to its end.
#include "q4_async.cuh"
#include <atomic>
#include <new>


namespace q4 {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_TN = 32;          // columns per CTA
// Workspace layout: a fixed 64 KiB head of arrival counters (one per column tile, so the
// counters of one shape never alias the partial sums of another), then the partial sums.
constexpr size_t GEMV_WS_HEAD = 131072;           // first half: arrival counters and the status word; second half: the
                                                  // exchange slots of the warp-specialised kernel (GEMV_WS_SLOTS)

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

// ---- sequential groups (group of row k = k / groupsize) and v1 layers: TMA streaming kernel --------
constexpr int GEMV_UNIT_ROWS = 32;                // packed rows per unit (256 k-rows, 8 steps)
constexpr int GEMV_UNIT_STEPS = GEMV_UNIT_ROWS / 4;
constexpr int GEMV_UNIT_BYTES = GEMV_UNIT_ROWS * GEMV_TN * 4;      // 4 KiB
constexpr int GEMV_META_ROWS = 9;                 // groups one unit can touch at groupsize 32, +1 straddle
constexpr int GEMV_SC_BYTES = 640;                // 9 rows x 32 halves, rounded up to 128
constexpr int GEMV_ZP_BYTES = 256;                // 9 rows x 16 B (v2) or 64 B of fp16 zeros (v1)
constexpr int GEMV_STAGE_BYTES = GEMV_UNIT_BYTES + GEMV_SC_BYTES + GEMV_ZP_BYTES;
constexpr int GEMV_WSTAGES = 2;                   // stages per warp
constexpr int GEMV_CWARPS = 16;
constexpr int GEMV_STREAM_THREADS = GEMV_CWARPS * 32;
constexpr int GEMV_XS_MAX_BYTES = 40960;          // largest x (+ its chunk table) kept in shared memory

struct GemvStreamParams {
  GemvParams g;
  int units_per_tile, total_units, steps_per_tile;
  int meta_rows;                                  // group rows fetched with each unit
  uint32_t stage_tx;                              // bytes TMA delivers per stage
  float* cta_part;                                // [grid][2][MT*8][32]
  unsigned* status;
  int group_shift;                                // log2(steps per group), or -1 if not a power of two
  unsigned long long* trace;                      // optional timing trace (64 slots per CTA), else null
  int whole_tiles;                                // lean kernel: CTAs get whole column tiles (no sums meet across CTAs)
  int n_groups;                                   // rows of scales / qzeros
  // lean kernel: what is dealt to the CTAs (`share` items of `per` units each) and the multipliers
  // ceil(2^32 / d) that turn its divisions by the grid size and by units_per_tile into one multiply
  // (exact while dividend * d < 2^32, which the host checks)
  unsigned share, per, magic_grid, magic_upt;
  // warp-specialised kernel: CTAs that have work (the grid may be larger: see launch_ws) and the word in the
  // workspace (after the head) through which they tell the spare CTAs that the launch is about to end
  int work_ctas;
  unsigned* leave_signal;
  unsigned long long* slots;                      // [CTA][32]: (partial sum, flag) words of a CTA's first, shared tile
  int prefetch_rows;                              // packed rows per L2 prefetch box (0: no prefetch)
  // the layer the caller will run next (q4_layer_set_next): its packed weights are asked into L2 while this
  // one computes; column tiles, boxes per tile and packed rows per box of that layer (0 rows: none)
  int next_tiles, next_bpt, next_rows;
};

template <int MT>
__host__ __device__ constexpr size_t gemv_stream_smem() {
  return (size_t)GEMV_CWARPS * GEMV_WSTAGES * GEMV_STAGE_BYTES + sizeof(float) * GEMV_CWARPS * MT * 8 * GEMV_TN +
         GEMV_CWARPS * GEMV_WSTAGES * 8 + 16;
}

__device__ __forceinline__ void trace_mark(unsigned long long* tr, int slot) {
  if (tr && slot < 64) tr[(size_t)blockIdx.x * 64 + slot] = clock64();
}
// the same with the device-wide nanosecond timer, to line up CTAs of different SMs and launches
__device__ __forceinline__ void trace_mark_ns(unsigned long long* tr, int slot) {
  if (tr && slot < 64) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    tr[(size_t)blockIdx.x * 64 + slot] = t;
  }
}

// CTA that owns unit u when `nu` units are dealt to `G` CTAs as [c*nu/G, (c+1)*nu/G).
__device__ __forceinline__ int unit_owner(long long u, int G, int nu) { return (int)(((u + 1) * G + nu - 1) / nu) - 1; }

// MMA whose accumulator starts at zero (first k-step of a group).
__device__ __forceinline__ void mma16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void named_bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// One CTA per SM, 16 warps, every warp an independent stream processor:
//   * qweight is cut into units of 32 packed rows x 32 columns (4 KiB = 256 k-rows x 32 outputs); the
//     units, ordered column tile by column tile, are dealt to the CTAs in equal contiguous runs
//     (stream-K) and inside a CTA round-robin to the warps.
//   * A warp fetches its own units with TMA (weights + the scale / zero-point rows the unit touches)
//     into a private two-stage ring and waits only on its own mbarriers, so in the steady state
//     there is no synchronisation between warps at all; for the LLaMA-7B shapes nearly every unit of
//     the launch is in flight within the first microsecond.
//   * At the end of a column tile every warp leaves its partial sums in shared memory and one warp
//     adds them (fixed order) and stores y, or hands a partial tile to the last CTA to arrive.
// FAST: the group size is a multiple of 128 rows (or the layer is v1), so each 128-row half of a unit
// lies in one group: no per-step group test.
// XS (needs FAST, M <= 8, K % 128 == 0, x + its table <= GEMV_XS_MAX_BYTES): x is copied once per CTA
// into shared memory in the order the MMA wants it, the odd k of every 8-block pre-divided by 16 so
// that the high nibble of each byte can be used where it sits (w & 0x00F000F0 | 0x6400 = 1024 + 16 q, no
// shift), and the per-128-row sums that take the 1024 / 64 offsets and the zero point out again are
// tabulated once.  That removes the x permutes, half of the shifts and the all-ones MMA from the loop.
template <int MT, bool FAST, bool XS>
__global__ void __launch_bounds__(GEMV_STREAM_THREADS, 1)
gemv_stream_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                   const __grid_constant__ CUtensorMap zmap, const GemvStreamParams sp) {
  extern __shared__ __align__(128) unsigned char smem[];
  const GemvParams& p = sp.g;
  constexpr int RED_FLOATS = GEMV_CWARPS * MT * 8 * GEMV_TN;
  float* red = reinterpret_cast<float*>(smem + (size_t)GEMV_CWARPS * GEMV_WSTAGES * GEMV_STAGE_BYTES);   // [16][MT*8][32]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + RED_FLOATS);                                         // [16][2]
  volatile int* flags = reinterpret_cast<volatile int*>(full + GEMV_CWARPS * GEMV_WSTAGES);              // [0] abort
  // XS only: [16 B of zeros][chunk table: K/128 x 8 float2][x rows, MMA order]
  unsigned char* xs_base = smem + gemv_stream_smem<MT>();
  float2* ctab = reinterpret_cast<float2*>(xs_base + 16);
  __half* xs_buf = reinterpret_cast<__half*>(xs_base + 16 + (size_t)(sp.g.K / 128) * 64);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nu = sp.total_units, G = gridDim.x, upt = sp.units_per_tile;
  const int u0 = (int)((long long)blockIdx.x * nu / G), u1 = (int)((long long)(blockIdx.x + 1) * nu / G);
  const int gs = p.groupsize;
  unsigned char* my_stages = smem + (size_t)warp * GEMV_WSTAGES * GEMV_STAGE_BYTES;
  uint64_t* my_full = full + warp * GEMV_WSTAGES;

  if (threadIdx.x == 0) {
    for (int i = 0; i < GEMV_CWARPS * GEMV_WSTAGES; ++i) mbar_init(&full[i], 1);
    flags[0] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&wmap); tma_prefetch_desc(&smap); tma_prefetch_desc(&zmap);
  }
  __syncthreads();
  pdl_launch_dependents();

  // Fetch this warp's n-th unit (CTA-local unit warp + 16 n) into stage n % 2: lanes 0..2 issue one copy each.
  auto issue = [&](int n) {
    const int u = u0 + warp + GEMV_CWARPS * n;
    if (u >= u1) return;
    const int tile = u / upt, ux = u - tile * upt;
    unsigned char* dst = my_stages + (size_t)(n % GEMV_WSTAGES) * GEMV_STAGE_BYTES;
    uint64_t* bar = &my_full[n % GEMV_WSTAGES];
    const int grow0 = p.v1 ? 0 : (ux * GEMV_UNIT_ROWS * 8) / gs;
    if (lane == 0) {
      mbar_arrive_expect_tx(bar, sp.stage_tx);
      tma_load_2d(dst, &wmap, tile * GEMV_TN, ux * GEMV_UNIT_ROWS, bar);
    } else if (lane == 1) {
      tma_load_2d(dst + GEMV_UNIT_BYTES, &smap, tile * GEMV_TN, grow0, bar);
    } else if (lane == 2) {
      tma_load_2d(dst + GEMV_UNIT_BYTES + GEMV_SC_BYTES, &zmap, p.v1 ? tile * GEMV_TN : tile * (GEMV_TN / 8), grow0, bar);
    }
  };
  issue(0);
  issue(1);                                              // weights never depend on an earlier kernel

  const int g = lane >> 2, t = lane & 3;
  const int K = p.K;
  const int steps_per_group = gs >> 5;
  const bool xok0 = g < p.M, xok1 = (g + 8) < p.M;
  const __half* xrow = p.x + (size_t)g * K + 8 * t;

  float yacc[MT][2][4];                                   // scaled sums of the closed groups of a tile
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) yacc[mt][j][i] = 0.f;

  // y += s * (acc - (1024 + z + 1) * xsum) for the group whose scales sit in row `grow` of the stage;
  // c / co are the raw MMA sums, one set per k-step parity so consecutive MMAs never wait on each other
  auto flush = [&](const unsigned char* stg, int grow, float (&c)[MT][2][2][4], float (&co)[MT][2][4], int chunk) {
    const uint2 sc = *reinterpret_cast<const uint2*>(stg + GEMV_UNIT_BYTES + grow * 64 + 8 * g);
    const float2 s01 = __half22float2(as_h2(sc.x)), s23 = __half22float2(as_h2(sc.y));
    const float s[4] = {s01.x, s01.y, s23.x, s23.y};
    float zz[4], zf[4];
    if (!p.v1) {
      const uint32_t zw = *reinterpret_cast<const uint32_t*>(stg + GEMV_UNIT_BYTES + GEMV_SC_BYTES + grow * 16 + 4 * (g >> 1));
      const uint32_t zb = zw >> (16 * (g & 1));
      // 1024 + z through the fp16 exponent trick: (z | 0x6400) is 1024 + z exactly
      const float2 za = __half22float2(as_h2(((zb & 0xFu) | ((zb & 0xF0u) << 12)) | 0x64006400u));
      const float2 zc = __half22float2(as_h2((((zb >> 8) & 0xFu) | ((zb & 0xF000u) << 4)) | 0x64006400u));
      const float off = XS ? -1023.f : 1.f;              // XS: plain z + 1, the offsets are in the table
      zz[0] = za.x + off; zz[1] = za.y + off; zz[2] = zc.x + off; zz[3] = zc.y + off;
#pragma unroll
      for (int i = 0; i < 4; ++i) zf[i] = 0.f;
    } else {          // W = s*q - zero: only the offsets scale with s, the float zero does not
      const uint2 zh = *reinterpret_cast<const uint2*>(stg + GEMV_UNIT_BYTES + GEMV_SC_BYTES + 8 * g);
      const float2 z01 = __half22float2(as_h2(zh.x)), z23 = __half22float2(as_h2(zh.y));
      zf[0] = z01.x; zf[1] = z01.y; zf[2] = z23.x; zf[3] = z23.y;
#pragma unroll
      for (int i = 0; i < 4; ++i) zz[i] = XS ? 0.f : 1024.f;
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float xs0, xs1, of0 = 0.f, of1 = 0.f;
      if constexpr (XS) {
        // table entry of batch column b: (1024*sum_even + 64*sum_odd, sum_even + sum_odd) of x over the chunk
        const float4 e = *reinterpret_cast<const float4*>(ctab + (size_t)chunk * 8 + 2 * t);
        of0 = e.x; xs0 = e.y; of1 = e.z; xs1 = e.w;
      } else {
        xs0 = co[mt][0][0] + co[mt][1][0]; xs1 = co[mt][0][1] + co[mt][1][1];
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = 2 * j + (i >> 1);
          const float xs = (i & 1) ? xs1 : xs0, of = (i & 1) ? of1 : of0;
          float v = fmaf(s[col], fmaf(-zz[col], xs, c[mt][j][0][i] + c[mt][j][1][i] - of), yacc[mt][j][i]);
          yacc[mt][j][i] = p.v1 ? fmaf(-zf[col], xs, v) : v;
        }
    }
  };

  // End of this CTA's run of units [seg_first, seg_last] in column tile `tile`.  Every warp leaves its
  // sums in `red`; only the last warp waits for the others, adds the 16 partials in warp order and
  // either stores y (the run covers the whole tile) or hands the tile's partial to the last CTA to arrive.
  //   named barrier 1: "red is complete"   (15 warps arrive, the reducer syncs)
  //   named barrier 2: "red may be reused" (the reducer arrives, 15 warps sync at the next tile)
  auto finish_tile = [&](int tile, int seq, int seg_first, int seg_last) {
    const bool reducer = warp == GEMV_CWARPS - 1;
    if (!reducer && seq >= 1) named_bar_sync(2, GEMV_STREAM_THREADS);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = 4 * g + 2 * j + (i >> 1), b = mt * 8 + 2 * t + (i & 1);
          red[(warp * (MT * 8) + b) * GEMV_TN + col] = yacc[mt][j][i];
          yacc[mt][j][i] = 0.f;
        }
    if (!reducer) {
      __threadfence_block();
      named_bar_arrive(1, GEMV_STREAM_THREADS);
      return;
    }
    named_bar_sync(1, GEMV_STREAM_THREADS);
    const int tc0 = tile * GEMV_TN, col = lane;
    const bool whole = seg_first == 0 && seg_last == upt - 1;
    const int c_first = unit_owner((long long)tile * upt, G, nu), c_last = unit_owner((long long)tile * upt + upt - 1, G, nu);
    // slot 0 of a CTA's partials: the run continues a tile begun by an earlier CTA; slot 1: it begins the tile
    float* part = sp.cta_part + ((size_t)blockIdx.x * 2 + (seg_first == 0 ? 1 : 0)) * (MT * 8) * GEMV_TN;
    for (int r = 0; r < p.M; ++r) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < GEMV_CWARPS; ++w) v += red[(w * (MT * 8) + r) * GEMV_TN + col];
      if (whole) store_y(p, r, tc0 + col, v);
      else __stcg(part + r * GEMV_TN + col, v);
    }
    named_bar_arrive(2, GEMV_STREAM_THREADS);
    if (whole) return;
    __threadfence();
    __syncwarp();
    unsigned last = 0;
    if (lane == 0) last = atomicAdd(p.counters + tile, 1u) == (unsigned)(c_last - c_first);
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    for (int r = 0; r < p.M; ++r) {
      float v = 0.f;
      // four contributors' partials in flight at a time, added in CTA order (an absent one adds +0)
      for (int cc = c_first; cc <= c_last; cc += 4) {
        float t4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          t4[i] = cc + i <= c_last ? __ldcg(sp.cta_part + ((size_t)(cc + i) * 2 + (cc + i == c_first ? 1 : 0)) * (MT * 8) * GEMV_TN + r * GEMV_TN + col) : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) v += t4[i];
      }
      store_y(p, r, tc0 + col, v);
    }
    if (lane == 0) p.counters[tile] = 0u;                // ready for the next launch
  };

  if (threadIdx.x == 0) trace_mark(sp.trace, 0);
  pdl_wait();                                            // x, y and the workspace belong to the stream order
  if (threadIdx.x == 0) trace_mark(sp.trace, 1);
  if constexpr (XS) {
    const int blocks_per_row = K >> 3;                   // 8-element blocks per x row, 16 per 128-row chunk
    if (threadIdx.x < 4) reinterpret_cast<uint32_t*>(xs_base)[threadIdx.x] = 0u;
    for (int idx = threadIdx.x; idx < (K >> 7) * 8; idx += GEMV_STREAM_THREADS)
      if ((idx & 7) >= p.M) ctab[idx] = make_float2(0.f, 0.f);
    // The trip count is the same for every lane of a warp (the sums below are full-warp shuffles): the
    // bound is rounded up to whole CTA strides and the lanes past the end carry zeros.  Rows are a
    // multiple of 16 blocks long, so the 16 lanes that share a sum always sit in one row and chunk.
    const int total = p.M * blocks_per_row;
    for (int base = 0; base < total; base += GEMV_STREAM_THREADS) {
      const int idx = base + threadIdx.x;
      const bool ok = idx < total;
      const int m = ok ? idx / blocks_per_row : 0, blk = ok ? idx - m * blocks_per_row : 0;
      const uint4 v = ok ? __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)m * K + 8 * blk)) : make_uint4(0u, 0u, 0u, 0u);
      const __half2 h01 = as_h2(v.x), h23 = as_h2(v.y), h45 = as_h2(v.z), h67 = as_h2(v.w);
      const __half2 sixteenth = as_h2(0x2C002C00u);
      const __half2 e04 = __lows2half2(h01, h45), o15 = __hmul2(__highs2half2(h01, h45), sixteenth);
      const __half2 e26 = __lows2half2(h23, h67), o37 = __hmul2(__highs2half2(h23, h67), sixteenth);
      if (ok) *reinterpret_cast<uint4*>(xs_buf + (size_t)m * K + 8 * blk) = make_uint4(as_u32(e04), as_u32(o15), as_u32(e26), as_u32(o37));
      const float2 f01 = __half22float2(h01), f23 = __half22float2(h23), f45 = __half22float2(h45), f67 = __half22float2(h67);
      float se = (f01.x + f23.x) + (f45.x + f67.x), so = (f01.y + f23.y) + (f45.y + f67.y);
#pragma unroll
      for (int d = 8; d >= 1; d >>= 1) { se += __shfl_xor_sync(0xffffffffu, se, d); so += __shfl_xor_sync(0xffffffffu, so, d); }
      // the odd elements sit in x' as x/16, so their 1024 offset comes back as 64 * x
      if (ok && (lane & 15) == 0) ctab[(size_t)(blk >> 4) * 8 + m] = make_float2(1024.f * se + 64.f * so, se + so);
    }
    named_bar_sync(5, GEMV_STREAM_THREADS);
  }
  if (threadIdx.x == 0) trace_mark(sp.trace, 2);

  // x of one 128-row half of a unit: four steps, rows 16*h .. 16*h+15 of the unit
  auto load_x = [&](uint4 (&xv)[MT][4], int ux, int h) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int stp = ux * GEMV_UNIT_STEPS + 4 * h + u;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const bool ok = (mt ? xok1 : xok0) && stp < sp.steps_per_tile;
        if constexpr (XS)
          xv[mt][u] = ok ? *reinterpret_cast<const uint4*>(xs_buf + (size_t)g * K + 8 * t + 32 * stp)
                         : *reinterpret_cast<const uint4*>(xs_base);
        else
          xv[mt][u] = ok ? __ldg(reinterpret_cast<const uint4*>(xrow + (size_t)(8 * mt) * K + 32 * stp))
                         : make_uint4(0, 0, 0, 0);
      }
    }
  };

  const int tile_first = u0 / upt, tile_last = (u1 - 1) / upt;
  int n = 0;                                             // index of this warp's next unit
  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int seg_u1 = min(u1, (tile + 1) * upt);
    for (int u = u0 + warp + GEMV_CWARPS * n; u < seg_u1; ++n, u += GEMV_CWARPS) {
      const int ux = u - tile * upt;
      const int st = n % GEMV_WSTAGES, use = n / GEMV_WSTAGES;
      uint4 xv[MT][4];
      load_x(xv, ux, 0);
      if (!mbar_wait_warp(&my_full[st], use & 1, flags[0] ? 4u : 20000u)) {
        flags[0] = 1; atomicExch(sp.status, Q4_STATUS_WAIT_EXPIRED);
      }
      if (warp == 0 && lane == 0) trace_mark(sp.trace, 3 + 2 * n);
      const unsigned char* stg = my_stages + (size_t)st * GEMV_STAGE_BYTES;
      const uint32_t* box = reinterpret_cast<const uint32_t*>(stg);
      const int grp0 = p.v1 ? 0 : (sp.group_shift >= 0 ? ((ux * GEMV_UNIT_STEPS) >> sp.group_shift) : (ux * GEMV_UNIT_ROWS * 8) / gs);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        if (h == 1) load_x(xv, ux, 1);
        const int step0 = ux * GEMV_UNIT_STEPS + 4 * h;
        if (step0 >= sp.steps_per_tile) break;           // rows past K were zero-filled by TMA
        uint4 wv[4];
#pragma unroll
        for (int uu = 0; uu < 4; ++uu)
          wv[uu] = *reinterpret_cast<const uint4*>(box + (4 * (4 * h + uu) + t) * GEMV_TN + 4 * g);
        float c[MT][2][2][4], co[MT][2][4];
        int cur_grp = -1;
        bool fresh = true;
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
          const int step = step0 + uu;
          if (step >= sp.steps_per_tile) break;
          if (!FAST) {
            const int grp = sp.group_shift >= 0 ? (step >> sp.group_shift) : step / steps_per_group;
            if (grp != cur_grp) {
              if (cur_grp >= 0) flush(stg, cur_grp - grp0, c, co, 0);
              cur_grp = grp; fresh = true;
            }
          }
          const uint32_t w[4] = {wv[uu].x, wv[uu].y, wv[uu].z, wv[uu].w};
          uint32_t pr[4][4];                      // pr[word][m] = (q_m, q_m+4) + 1024  (XS, odd m: 16 q + 1024)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if constexpr (XS) {
              const uint32_t w8 = w[q] >> 8;
              pr[q][0] = and_or(w[q], 0x000F000Fu, 0x64006400u);
              pr[q][1] = and_or(w[q], 0x00F000F0u, 0x64006400u);
              pr[q][2] = and_or(w8, 0x000F000Fu, 0x64006400u);
              pr[q][3] = and_or(w8, 0x00F000F0u, 0x64006400u);
            } else {
              pr[q][0] = and_or(w[q], 0x000F000Fu, 0x64006400u);
              pr[q][1] = and_or(w[q] >> 4, 0x000F000Fu, 0x64006400u);
              pr[q][2] = and_or(w[q] >> 8, 0x000F000Fu, 0x64006400u);
              pr[q][3] = and_or(w[q] >> 12, 0x000F000Fu, 0x64006400u);
            }
          }
          const bool first = FAST ? (uu == 0) : fresh;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 xq = xv[mt][uu];            // x[k..k+7] of batch row g (+8); XS: already in MMA order
            uint32_t xb[4];
            if constexpr (XS) {
              xb[0] = xq.x; xb[1] = xq.y; xb[2] = xq.z; xb[3] = xq.w;
            } else {
              xb[0] = prmt(xq.x, xq.z, 0x5410); xb[1] = prmt(xq.x, xq.z, 0x7632);    // (x0,x4) (x1,x5)
              xb[2] = prmt(xq.y, xq.w, 0x5410); xb[3] = prmt(xq.y, xq.w, 0x7632);    // (x2,x6) (x3,x7)
            }
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              const uint32_t bb0 = xb[2 * ks], bb1 = xb[2 * ks + 1];
              if (first) {
                mma16816_first(c[mt][0][ks], pr[0][2 * ks], pr[1][2 * ks], pr[0][2 * ks + 1], pr[1][2 * ks + 1], bb0, bb1);
                mma16816_first(c[mt][1][ks], pr[2][2 * ks], pr[3][2 * ks], pr[2][2 * ks + 1], pr[3][2 * ks + 1], bb0, bb1);
                if constexpr (!XS) mma16816_first(co[mt][ks], 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, bb0, bb1);
              } else {
                mma16816(c[mt][0][ks], pr[0][2 * ks], pr[1][2 * ks], pr[0][2 * ks + 1], pr[1][2 * ks + 1], bb0, bb1);
                mma16816(c[mt][1][ks], pr[2][2 * ks], pr[3][2 * ks], pr[2][2 * ks + 1], pr[3][2 * ks + 1], bb0, bb1);
                if constexpr (!XS) mma16816(co[mt][ks], 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, bb0, bb1);
              }
            }
          }
          fresh = false;
        }
        // scales live in this stage: settle the open group before the stage is refilled
        if (FAST) {
          flush(stg, p.v1 ? 0 : ((sp.group_shift >= 0 ? (step0 >> sp.group_shift) : step0 / steps_per_group) - grp0), c, co, step0 >> 2);
        } else if (cur_grp >= 0) {
          flush(stg, cur_grp - grp0, c, co, 0);
        }
      }
      __syncwarp();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // our reads before the next TMA write
      issue(n + GEMV_WSTAGES);
      if (warp == 0 && lane == 0) trace_mark(sp.trace, 4 + 2 * n);
    }
    if (threadIdx.x == 0) trace_mark(sp.trace, 30);
    finish_tile(tile, tile - tile_first, max(u0, tile * upt) - tile * upt, seg_u1 - 1 - tile * upt);
    if (threadIdx.x == 0) trace_mark(sp.trace, 31);
  }
}

// ---- M <= 8, sequential groups of a multiple of 128 rows: the lean decode kernel --------------------
// Same decomposition as gemv_stream_kernel (independent per-warp TMA streams over 4 KiB units), with
// everything per-step stripped to the minimum:
//   * x of a unit (256 halves per batch row) arrives in the warp's stage with cp.async next to the
//     weights and is rewritten in place into MMA order, odd elements divided by 16, so the B fragment of
//     a step is one LDS.128 and the high nibbles of the packed words are used where they sit
//     (w & 0x00F000F0 | 0x6400 = 1024 + 16 q): 5 integer instructions per 8 weights.
//   * the +1024 / +64 offsets and the zero points are not handled per MMA fragment: one lane per
//     column subtracts s * (offset_sum + (z+1) * x_sum) once per group, from sums of x computed once
//     per unit with warp shuffles.
// Warps per CTA (W) and CTAs per SM (OCC) are parameters of the kernel.  With one CTA per SM (W = 16, or 12
// where the stages of 16 - 4 KiB of weights + MR x 512 B of x each - do not fit) the CTAs of the next launch
// in the stream cannot become resident before this launch's CTAs exit, so its prologue and its first weight
// copies start only then.  The two-per-SM form (fewer warps, at most half of the SM's shared memory and
// registers per CTA) leaves room for them: the next launch's CTAs start, issue their first weight copies and
// park in griddepcontrol.wait while this launch is still streaming.
constexpr int GF_STAGES = 2;
// A stage is two blocks.  The packed words (4 KiB, TMA with the 128-byte swizzle: the 16-byte chunk c of
// row r lies at chunk c ^ (r & 7), which needs the block on a 1 KiB boundary) and, in a ring of its own,
// the small operands of the unit:
constexpr int GF_META_OFF = 0;                        // scales: 2 rows x 64 B
constexpr int GF_ZP_OFF = GF_META_OFF + 128;          // zero points: 2 rows x 16 B
constexpr int GF_X_OFF = GF_ZP_OFF + 128;             // x: MR rows of 512 B at a pitch of 528 B, then the sums: 2 chunks x MR x float2
constexpr int GF_X_PITCH = 528;                       // odd multiple of 16 B: the rows of a quarter-warp's loads fall on different banks

template <int MR>
__host__ __device__ constexpr int gf_aux_bytes(bool xc) { return xc ? GF_X_OFF : (GF_X_OFF + MR * GF_X_PITCH + 64 + 127) / 128 * 128; }
// With XC the whole of x is re-laid out once per CTA instead of per unit: x' rows of `xc_pitch` bytes
// (k padded to whole units, plus 16 so that neighbouring rows start on different banks) and one
// (offset sum, plain sum) pair per 128 k and row.
__host__ __device__ inline size_t gf_xc_bytes(int mr, int upt) { return (size_t)mr * (upt * 512 + 16) + (size_t)upt * 2 * mr * 8; }
template <int MR, int W>
__host__ __device__ constexpr size_t gf_smem_bytes(bool xc) {
  return 1024 + (size_t)W * GF_STAGES * (GEMV_UNIT_BYTES + gf_aux_bytes<MR>(xc)) + sizeof(float) * W * MR * GEMV_TN +
         W * GF_STAGES * 8 + 64;
}

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async16_zfill_if(bool pred, void* dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %3, 0;\n\t@p cp.async.ca.shared.global [%0], [%1], 16, %2;\n\t}"
               ::"r"(smem_u32(dst)), "l"(src), "r"(n), "r"((uint32_t)pred) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// TRACE: the instance that records timestamps (q4_gemv_set_trace); the other carries no trace code at all
// V1: the first layer format - one scale and one fp16 zero term per column (W = s q - zero), no groups
template <int MR, bool TRACE, bool XC, bool V1, int W, int OCC>
__global__ void __launch_bounds__(W * 32, OCC)
gemv_fast_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                 const __grid_constant__ CUtensorMap zmap, const GemvStreamParams sp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);            // the swizzle works on address bits
  const GemvParams& p = sp.g;
  unsigned long long* const trc = TRACE ? sp.trace : nullptr;
  constexpr int STG = GEMV_UNIT_BYTES, AUX = gf_aux_bytes<MR>(XC);
  constexpr int GF_WARPS = W, GF_THREADS = GF_WARPS * 32;
  unsigned char* aux_ring = smem + (size_t)GF_WARPS * GF_STAGES * STG;
  unsigned char* xc = aux_ring + (size_t)GF_WARPS * GF_STAGES * AUX;                            // XC: x' of the whole layer
  const int xc_pitch = sp.units_per_tile * 512 + 16;
  float2* xc_sums = reinterpret_cast<float2*>(xc + (size_t)MR * xc_pitch);                       // XC: [K / 128][MR]
  float* red = reinterpret_cast<float*>(xc + (XC ? gf_xc_bytes(MR, sp.units_per_tile) : 0));    // [16][MR][32]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + GF_WARPS * MR * GEMV_TN);                  // [16][2]
  volatile int* flags = reinterpret_cast<volatile int*>(full + GF_WARPS * GF_STAGES);          // [0] abort

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) trace_mark_ns(trc, 40);
  const int nu = sp.total_units, G = gridDim.x, upt = sp.units_per_tile;
  // this CTA's units [u0, u1): an even share of all units, or (whole_tiles) of all column tiles
  // (the host keeps nu * G below 2^32, so 32-bit arithmetic is exact)
  const unsigned share = sp.share, per = sp.per;
  const int u0 = (int)(__umulhi((unsigned)blockIdx.x * share, sp.magic_grid) * per);
  const int u1 = (int)(__umulhi(((unsigned)blockIdx.x + 1u) * share, sp.magic_grid) * per);
  const int K = p.K, gs = p.groupsize;
  unsigned char* my_stages = smem + (size_t)warp * GF_STAGES * STG;
  unsigned char* my_aux = aux_ring + (size_t)warp * GF_STAGES * AUX;
  uint64_t* my_full = full + warp * GF_STAGES;

  if (lane < GF_STAGES) {                                 // every warp sets up its own barriers
    mbar_init(&my_full[lane], 1 + 32);                    // TMA arrive + 32 cp.async arrivals
    mbar_fence_init();
  }
  if (threadIdx.x == 0) {
    flags[0] = 0;
    tma_prefetch_desc(&wmap); tma_prefetch_desc(&smap); tma_prefetch_desc(&zmap);
  }
  if (threadIdx.x == 0) trace_mark_ns(trc, 46);
  __syncthreads();
  if (threadIdx.x == 0) trace_mark_ns(trc, 47);
  pdl_launch_dependents();

  // The warp's units are u0 + warp + 16 n, n = 0, 1, ...; both issue streams below walk them in
  // order and keep (tile, unit within tile) by stepping, so that no unit costs an integer division.
  struct Cursor { int u, tile, ux; };
  auto cursor_step = [&](Cursor& c) {
    c.u += GF_WARPS; c.ux += GF_WARPS;
    while (c.ux >= upt) { c.ux -= upt; ++c.tile; }
  };
  Cursor cw, cx;
  cw.u = u0 + warp; cw.tile = (int)__umulhi((unsigned)cw.u, sp.magic_upt); cw.ux = cw.u - cw.tile * upt;
  cx = cw;
  // packed weights of this warp's n-th unit: one TMA copy, issued by lane 0
  auto issue_w = [&](int n) {
    if (cw.u >= u1) return;
    tma_expect_load_2d_if(lane == 0, my_stages + (size_t)(n % GF_STAGES) * STG, &wmap, cw.tile * GEMV_TN, cw.ux * GEMV_UNIT_ROWS,
                          &my_full[n % GF_STAGES], GEMV_UNIT_BYTES);
    cursor_step(cw);
  };
  // x of the same unit (every lane copies its 8 elements of every batch row) and, on lanes 0..9, the
  // unit's two group rows of scales (4 x 16 bytes each) and of packed zero points (16 bytes each);
  // then every lane arrives on the barrier.  One TMA copy per unit instead of three: issuing a
  // TMA copy occupies the issuing thread for some 200 cycles, an asynchronous 16-byte copy does not.
  // lanes 0..7 copy 16 bytes of one of the unit's two scale rows, lanes 8 and 9 one of its two zero-point rows
  // (V1: lanes 0..3 the one scale row, lanes 8..11 the 64 bytes of fp16 zero terms of the tile's 32 columns)
  const bool meta_lane = lane < (V1 ? 12 : 10);
  const int meta_sel = lane < 8 ? (lane >> 2) : (V1 ? 0 : lane - 8);
  const unsigned char* meta_src = lane < 8 ? reinterpret_cast<const unsigned char*>(p.scales + 8 * (lane & 3))
                                : V1       ? reinterpret_cast<const unsigned char*>(p.qzeros) + 16 * (lane - 8)
                                           : reinterpret_cast<const unsigned char*>(p.qzeros);
  const size_t meta_pitch = lane < 8 ? (size_t)p.N * 2 : (size_t)(p.N >> 3) * 4;        // bytes per group row
  const int meta_tile = (lane < 8 || V1) ? GEMV_TN * 2 : (GEMV_TN / 8) * 4;              // bytes per column tile
  const int meta_dst = lane < 8 ? GF_META_OFF + 16 * lane : GF_ZP_OFF + 16 * (lane - 8);
  auto issue_x = [&](int n) {
    if (cx.u >= u1) return;
    unsigned char* stg = my_aux + (size_t)(n % GF_STAGES) * AUX;
    unsigned char* dst = stg + GF_X_OFF;
    if constexpr (!XC) {
      const int k = cx.ux * 256 + 8 * lane;
#pragma unroll
      for (int r = 0; r < MR; ++r)
        cp_async16_zfill(dst + r * GF_X_PITCH + 16 * lane, p.x + (size_t)(r < p.M ? r : 0) * K + (k < K ? k : 0), r < p.M && k < K);
    }
    {
      // lanes 10..31 run the same address arithmetic and copy nothing (a predicated copy, not a branch)
      const int grow0 = sp.group_shift >= 0 ? ((cx.ux * GEMV_UNIT_STEPS) >> sp.group_shift) : (cx.ux * GEMV_UNIT_ROWS * 8) / gs;
      const int row = grow0 + meta_sel;
      const bool ok = row < sp.n_groups;
      cp_async16_zfill_if(meta_lane, stg + meta_dst, meta_src + (size_t)(ok ? row : 0) * meta_pitch + cx.tile * meta_tile, ok);
    }
    cp_async_arrive_noinc(&my_full[n % GF_STAGES]);
    cursor_step(cx);
  };
  // inside the unit loop both copies of a unit are issued together and one cursor serves both
  auto issue_wx = [&](int n) {
    if (cw.u >= u1) return;
    cx = cw;
    issue_w(n);
    issue_x(n);
  };
  if (threadIdx.x == 0) trace_mark_ns(trc, 48);
  issue_w(0);
  issue_w(1);                                            // weights never depend on an earlier kernel
  if (threadIdx.x == 0) trace_mark_ns(trc, 41);
  pdl_wait();                                            // x, y and the workspace belong to the stream order
  if (threadIdx.x == 0) trace_mark_ns(trc, 42);
  issue_x(0);
  issue_x(1);
  if constexpr (XC) {
    // x' of all rows and the sums of every 128 k, once for the CTA: 16 lanes share one 128-k chunk
    const int blocks = sp.units_per_tile * 32;           // 8-element blocks per padded row (a multiple of 16)
    for (int idx = threadIdx.x; idx < MR * blocks; idx += GF_THREADS) {
      const int m = idx / blocks, blk = idx - m * blocks;
      const bool ok = m < p.M && 8 * blk < K;
      const uint4 v = ok ? __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)m * K + 8 * blk)) : make_uint4(0u, 0u, 0u, 0u);
      const __half2 h01 = as_h2(v.x), h23 = as_h2(v.y), h45 = as_h2(v.z), h67 = as_h2(v.w);
      const __half2 sixteenth = as_h2(0x2C002C00u);
      const __half2 e04 = __lows2half2(h01, h45), o15 = __hmul2(__highs2half2(h01, h45), sixteenth);
      const __half2 e26 = __lows2half2(h23, h67), o37 = __hmul2(__highs2half2(h23, h67), sixteenth);
      *reinterpret_cast<uint4*>(xc + (size_t)m * xc_pitch + 16 * blk) = make_uint4(as_u32(e04), as_u32(o15), as_u32(e26), as_u32(o37));
      const float2 f01 = __half22float2(h01), f23 = __half22float2(h23), f45 = __half22float2(h45), f67 = __half22float2(h67);
      float se = (f01.x + f23.x) + (f45.x + f67.x), so = (f01.y + f23.y) + (f45.y + f67.y);
#pragma unroll
      for (int d = 8; d >= 1; d >>= 1) { se += __shfl_xor_sync(0xffffffffu, se, d); so += __shfl_xor_sync(0xffffffffu, so, d); }
      if ((lane & 15) == 0) xc_sums[(blk >> 4) * MR + m] = make_float2(1024.f * se + 64.f * so, se + so);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) trace_mark(trc, 0);

  const int g = lane >> 2, t = lane & 3;
  // Packed words: lane (g, t) takes columns 4g..4g+3 of rows 2t (+1) of every block of eight rows.  With
  // the rows a quarter-warp reads two apart, the swizzle puts its eight 16-byte chunks on eight different
  // bank groups (rows t, t+1, ... at chunk g would put them on two).
  const uint32_t woff0 = 128u * (2 * t) + 16u * (g ^ (2 * t)), woff1 = 128u * (2 * t + 1) + 16u * (g ^ (2 * t + 1));
  float yacc[2][4], ycorr[MR];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) yacc[j][i] = 0.f;
#pragma unroll
  for (int r = 0; r < MR; ++r) ycorr[r] = 0.f;

  auto finish_tile = [&](int tile, int seq, int seg_first, int seg_last) {
    const bool reducer = warp == GF_WARPS - 1;
    if (!reducer && seq >= 1) named_bar_sync(2, GF_THREADS);
    float* mine = red + warp * MR * GEMV_TN;
    if (2 * t < MR) {                                    // batch rows 2t and 2t + 1 live in the lanes with this t
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (2 * t + (i & 1) < MR) mine[(2 * t + (i & 1)) * GEMV_TN + 4 * g + 2 * j + (i >> 1)] = yacc[j][i];
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) yacc[j][i] = 0.f;
    __syncwarp();
#pragma unroll
    for (int r = 0; r < MR; ++r) { mine[r * GEMV_TN + lane] -= ycorr[r]; ycorr[r] = 0.f; }
    if (!reducer) {
      __threadfence_block();
      named_bar_arrive(1, GF_THREADS);
      return;
    }
    named_bar_sync(1, GF_THREADS);
    const int tc0 = tile * GEMV_TN, col = lane;
    const bool whole = seg_first == 0 && seg_last == upt - 1;
    float* part = sp.cta_part + ((size_t)blockIdx.x * 2 + (seg_first == 0 ? 1 : 0)) * 16 * GEMV_TN;
    for (int r = 0; r < p.M; ++r) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < GF_WARPS; ++w) v += red[(w * MR + r) * GEMV_TN + col];
      if (whole) store_y(p, r, tc0 + col, v);
      else __stcg(part + r * GEMV_TN + col, v);
    }
    named_bar_arrive(2, GF_THREADS);
    if (whole) return;
    const int c_first = unit_owner((long long)tile * upt, G, nu), c_last = unit_owner((long long)tile * upt + upt - 1, G, nu);
    __threadfence();
    __syncwarp();
    unsigned last = 0;
    if (lane == 0) last = atomicAdd(p.counters + tile, 1u) == (unsigned)(c_last - c_first);
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    for (int r = 0; r < p.M; ++r) {
      float v = 0.f;
      // four contributors' partials in flight at a time, added in CTA order (an absent one adds +0)
      for (int cc = c_first; cc <= c_last; cc += 4) {
        float t4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          t4[i] = cc + i <= c_last ? __ldcg(sp.cta_part + ((size_t)(cc + i) * 2 + (cc + i == c_first ? 1 : 0)) * 16 * GEMV_TN + r * GEMV_TN + col) : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) v += t4[i];
      }
      store_y(p, r, tc0 + col, v);
    }
    if (lane == 0) p.counters[tile] = 0u;
  };

  const int tile_first = (int)__umulhi((unsigned)u0, sp.magic_upt), tile_last = (int)__umulhi((unsigned)(u1 - 1), sp.magic_upt);
  int n = 0;
  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int seg_u1 = min(u1, (tile + 1) * upt);
    for (int u = u0 + warp + GF_WARPS * n; u < seg_u1; ++n, u += GF_WARPS) {
      const int ux = u - tile * upt;
      const int st = n % GF_STAGES, use = n / GF_STAGES;
      if (!mbar_test_wait(&my_full[st], use & 1)) {
        // not there yet: every lane tests the barrier itself (one instruction per try, no vote or shuffle
        // afterwards), up to a limit that shrinks once any wait of the CTA has expired
        uint32_t tries = 0;
        const uint32_t lim = flags[0] ? 64u : 20000000u;
        while (!mbar_test_wait(&my_full[st], use & 1) && ++tries < lim) {}
        if (tries >= lim) { flags[0] = 1; atomicExch(sp.status, Q4_STATUS_WAIT_EXPIRED); }
      }
      if (warp == 0 && lane == 0) trace_mark(trc, 3 + 2 * n);
      if (warp == 0 && lane == 0 && n == 0) trace_mark_ns(trc, 43);
      const unsigned char* wst = my_stages + (size_t)st * STG;
      unsigned char* stg = my_aux + (size_t)st * AUX;
      // ---- x: rewrite this lane's 8 elements per batch row in MMA order, and the unit's sums of x ----
      // (XC: both are in the CTA's x' already)
      float2* sums = XC ? xc_sums + 2 * ux * MR : reinterpret_cast<float2*>(stg + GF_X_OFF + MR * GF_X_PITCH);      // [2 chunks][MR]
#pragma unroll
      for (int r = 0; r < (XC ? 0 : MR); ++r) {
        uint4* px = reinterpret_cast<uint4*>(stg + GF_X_OFF + r * GF_X_PITCH + 16 * lane);
        const uint4 v = *px;
        const __half2 h01 = as_h2(v.x), h23 = as_h2(v.y), h45 = as_h2(v.z), h67 = as_h2(v.w);
        const __half2 sixteenth = as_h2(0x2C002C00u);
        const __half2 e04 = __lows2half2(h01, h45), o15 = __hmul2(__highs2half2(h01, h45), sixteenth);
        const __half2 e26 = __lows2half2(h23, h67), o37 = __hmul2(__highs2half2(h23, h67), sixteenth);
        *px = make_uint4(as_u32(e04), as_u32(o15), as_u32(e26), as_u32(o37));
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23), f45 = __half22float2(h45), f67 = __half22float2(h67);
        float se = (f01.x + f23.x) + (f45.x + f67.x), so = (f01.y + f23.y) + (f45.y + f67.y);
#pragma unroll
        for (int d = 8; d >= 1; d >>= 1) { se += __shfl_xor_sync(0xffffffffu, se, d); so += __shfl_xor_sync(0xffffffffu, so, d); }
        // odd elements sit in x' as x/16: their 1024 offset comes back as 64 x
        if ((lane & 15) == 0) sums[(lane >> 4) * MR + r] = make_float2(1024.f * se + 64.f * so, se + so);
      }
      if constexpr (!XC) __syncwarp();
      if (warp == 0 && lane == 0 && n < 2) trace_mark(trc, 50 + 5 * n);
      // lanes of batch rows that do not exist feed row 0 again: an MMA output column depends on its own
      // input column only, and the columns beyond MR are never stored
      const uint4* xq = XC ? reinterpret_cast<const uint4*>(xc + (size_t)(g < MR ? g : 0) * xc_pitch + 512 * ux) + 2 * t
                           : reinterpret_cast<const uint4*>(stg + GF_X_OFF + (g < MR ? g : 0) * GF_X_PITCH) + 2 * t;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float c[2][4];                                  // raw sums of the half: columns 4g, 4g+1 | 4g+2, 4g+3
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
          // step (h, uu) takes packed rows 8 j + 2 t + pp of the unit, j = 2 h + uu / 2, pp = uu & 1
          const uint4 wv = *reinterpret_cast<const uint4*>(wst + ((uu & 1) ? woff1 : woff0) + 1024 * (2 * h + (uu >> 1)));
          const uint4 xv = xq[8 * (2 * h + (uu >> 1)) + (uu & 1)];
          const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
          uint32_t pr[4][4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t w8 = w[q] >> 8;
            pr[q][0] = and_or(w[q], 0x000F000Fu, 0x64006400u);
            pr[q][1] = and_or(w[q], 0x00F000F0u, 0x64006400u);
            pr[q][2] = and_or(w8, 0x000F000Fu, 0x64006400u);
            pr[q][3] = and_or(w8, 0x00F000F0u, 0x64006400u);
          }
          if (uu == 0) {
            mma16816_first(c[0], pr[0][0], pr[1][0], pr[0][1], pr[1][1], xv.x, xv.y);
            mma16816_first(c[1], pr[2][0], pr[3][0], pr[2][1], pr[3][1], xv.x, xv.y);
          } else {
            mma16816(c[0], pr[0][0], pr[1][0], pr[0][1], pr[1][1], xv.x, xv.y);
            mma16816(c[1], pr[2][0], pr[3][0], pr[2][1], pr[3][1], xv.x, xv.y);
          }
          mma16816(c[0], pr[0][2], pr[1][2], pr[0][3], pr[1][3], xv.z, xv.w);
          mma16816(c[1], pr[2][2], pr[3][2], pr[2][3], pr[3][3], xv.z, xv.w);
        }
        // close the group of this half: scale the raw sums, and (one lane per column) take the offsets
        // and the zero point out: y -= s * (offset_sum + (z + 1) * x_sum)
        const int grow = (h == 1 && gs == 128) ? 1 : 0;            // gs = 128: two groups per unit; else the second
                                                                   // half only starts a new group at a unit boundary
        const uint2 sc = *reinterpret_cast<const uint2*>(stg + GF_META_OFF + grow * 64 + 8 * g);
        const float2 s01 = __half22float2(as_h2(sc.x)), s23 = __half22float2(as_h2(sc.y));
        yacc[0][0] = fmaf(s01.x, c[0][0], yacc[0][0]);
        yacc[0][1] = fmaf(s01.x, c[0][1], yacc[0][1]);
        yacc[0][2] = fmaf(s01.y, c[0][2], yacc[0][2]);
        yacc[0][3] = fmaf(s01.y, c[0][3], yacc[0][3]);
        yacc[1][0] = fmaf(s23.x, c[1][0], yacc[1][0]);
        yacc[1][1] = fmaf(s23.x, c[1][1], yacc[1][1]);
        yacc[1][2] = fmaf(s23.y, c[1][2], yacc[1][2]);
        yacc[1][3] = fmaf(s23.y, c[1][3], yacc[1][3]);
        const float sl = __half2float(*reinterpret_cast<const __half*>(stg + GF_META_OFF + grow * 64 + 2 * lane));
        if constexpr (V1) {
          const float zf = __half2float(*reinterpret_cast<const __half*>(stg + GF_ZP_OFF + 2 * lane));
#pragma unroll
          for (int r = 0; r < MR; ++r) {
            const float2 e = sums[h * MR + r];
            ycorr[r] = fmaf(zf, e.y, fmaf(sl, e.x, ycorr[r]));       // y -= s * offset_sum + zero * x_sum
          }
        } else {
          const uint32_t zw = *reinterpret_cast<const uint32_t*>(stg + GF_ZP_OFF + grow * 16 + 4 * (lane >> 3));
          const float z1 = (float)(((zw >> (4 * (lane & 7))) & 0xFu) + 1u);
#pragma unroll
          for (int r = 0; r < MR; ++r) {
            const float2 e = sums[h * MR + r];
            ycorr[r] = fmaf(sl, fmaf(z1, e.y, e.x), ycorr[r]);
          }
        }
        if (warp == 0 && lane == 0 && n < 2) trace_mark(trc, 51 + 5 * n + h);
      }
      __syncwarp();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // our reads before the next TMA write
      if (warp == 0 && lane == 0 && n < 2) trace_mark(trc, 53 + 5 * n);
      issue_wx(n + GF_STAGES);
      if (warp == 0 && lane == 0) trace_mark(trc, 4 + 2 * n);
    }
    if (threadIdx.x == 0) trace_mark(trc, 30);
    if (warp == GF_WARPS - 1 && lane == 0 && tile == tile_last) trace_mark_ns(trc, 44);
    finish_tile(tile, tile - tile_first, max(u0, tile * upt) - tile * upt, seg_u1 - 1 - tile * upt);
    if (threadIdx.x == 0) trace_mark(trc, 31);
    if (warp == GF_WARPS - 1 && lane == 0 && tile == tile_last) trace_mark_ns(trc, 45);
  }
}

// ---- one row, groups of 128: the warp-specialised decode kernel ------------------------------------
// What the measurements on a B200 said about the lean kernel above, and what this kernel does about it:
//   * With every weight byte already in L2 a launch is hardly faster than from HBM: the one-row product is
//     bound by instruction issue and by the latency chain of a launch, not by memory.  The non-tensor pipes
//     issue one warp instruction per two cycles per scheduler (LOP3, SHF, PRMT, IMAD, HFMA2 alike), the legacy
//     mma.sync path one m16n8k16 per 8 cycles; unpacking to fp16 costs 5 integer instructions per 8 weights.
//     Here the packed words are split into bytes, not halves: w & 0x0F0F0F0F and (w >> 4) & 0x0F0F0F0F are the
//     eight levels of a word as two u8x4 operands of mma.sync.m16n8k32 (3 instructions per 8 weights, and half
//     as many MMAs per weight).  x is converted once per CTA to 16-bit block fixed point - per group of 128
//     rows x_int = rn(x * 2^(14 - E)), 2^E <= max |x| of the group - and enters as two byte digits
//     (x_int = 256 hi + lo, hi signed, lo unsigned).  Products and sums are exact integers; the zero point
//     leaves through the exact integer sum of the group's x_int; the only rounding of the whole product is
//     that of x itself: none for elements within a factor 16 of their group's largest, an absolute error of at
//     most 2^(E-15) for the smaller ones.
//   * A warp of the lean kernel spent a fifth of its time per unit re-laying x out and a fifth issuing its
//     next copies.  Here the consumers convert x once, together, while the first weights are still on their
//     way, and refills are issued by a warp of their own (lane c for consumer c: issued one after the other
//     by one thread a copy costs 300 cycles, issued side by side by the lanes of one instruction under 100).
//   * Every consumer sets up its own two barriers and issues its own first copies, so that the launch's
//     copies are all under way a few hundred cycles after the CTA starts.
// Roles: warps 0..W-1 consume; warp W issues the metadata boxes (scales and packed zero points of all groups
// of a column tile, one TMA box each), the L2 prefetches and the refills.  Stage ring per consumer: S units
// of 4 KiB (TMA, 128-byte swizzle).  Two shapes of the kernel: W = 16, one CTA per SM; W = 8 at less than half
// of the SM's shared memory and registers, so that the next decode launch of the stream becomes resident
// beside this one and fills its rings while this one computes.
constexpr int WS_MAX_UNITS_PER_TILE = 256;             // K <= 65536

struct WsLayout {                                      // byte offsets from the 1 KiB-aligned base
  int stages, meta, meta_slot, meta_zp, xp, xinfo, red, bars, total;
};
__host__ __device__ inline WsLayout ws_layout(int W, int S, int G, int upt) {
  WsLayout l;
  l.stages = 0;
  l.meta = W * S * GEMV_UNIT_BYTES;
  l.meta_zp = (G * 64 + 127) / 128 * 128;              // scales [G][32] fp16, then zero points [G][4] words
  l.meta_slot = l.meta_zp + (G * 16 + 127) / 128 * 128;
  l.xp = l.meta + 2 * l.meta_slot;
  l.xinfo = l.xp + upt * 512;                          // x digits: 16 bytes per 8 k
  l.red = l.xinfo + upt * 16;                          // per 128 k: (2^(E-14), sum of x_int)
  l.bars = (l.red + W * GEMV_TN * 4 + 15) / 16 * 16;
  l.total = l.bars + 8 * (2 * W * S + 5) + 16 + 128;       // + the barrier and the 32 sums of the exchange
  return l;
}

__device__ __forceinline__ bool mbar_wait_sleep_bounded(uint64_t* bar, uint32_t parity, uint32_t tries) {
  for (uint32_t i = 0; i < tries; ++i)
    if (mbar_try_wait_sleep(bar, parity, 1000u)) return true;
  return false;
}
// every lane polls (one instruction per try); returns false when the limit ran out
__device__ __forceinline__ bool mbar_spin_bounded(uint64_t* bar, uint32_t parity, uint32_t tries) {
  if (mbar_test_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < tries; ++i)
    if (mbar_test_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void named_bar_sync_all(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// D += A (u8, 16 x 32) * B (s8 or u8, 32 x 8), s32 accumulators
__device__ __forceinline__ void imma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_u8u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// the same with the accumulators starting at zero (first step of a group)
__device__ __forceinline__ void imma_u8s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_u8u8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <int W, int S, int OCC, bool TRACE>
__global__ void __launch_bounds__((W + 2) * 32, OCC)
gemv_ws_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
               const __grid_constant__ CUtensorMap zmap, const __grid_constant__ CUtensorMap pmap,
               const __grid_constant__ CUtensorMap nmap, const GemvStreamParams sp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const GemvParams& p = sp.g;
  unsigned long long* const trc = TRACE ? sp.trace : nullptr;
  const int upt = sp.units_per_tile, G = sp.n_groups;
  const WsLayout L = ws_layout(W, S, G, upt);
  unsigned char* xp = smem + L.xp;                                   // digits of x_int: 16 bytes per 8 k
  float2* xinfo = reinterpret_cast<float2*>(smem + L.xinfo);         // [K / 128]: (2^(E-14), sum of x_int)
  float* red = reinterpret_cast<float*>(smem + L.red);               // [W][32]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);       // [W][S]  unit has landed
  uint64_t* empty = full + W * S;                                    // [W][S]  unit has been consumed
  uint64_t* mfull = empty + W * S;                                   // [2]     metadata of a tile has landed
  uint64_t* mempty = mfull + 2;                                      // [2]     every consumer is done with it
  uint64_t* rfull = mempty + 2;                                      // [1]     the other CTAs' sums of the owned tile are here
  volatile int* flags = reinterpret_cast<volatile int*>(rfull + 1);
  float* remote = reinterpret_cast<float*>(rfull + 3);               // [32]
  constexpr int ALL = (W + 2) * 32, CT = W * 32;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) trace_mark_ns(trc, 40);
  const int nu = sp.total_units, Gd = sp.work_ctas;
  if ((int)blockIdx.x >= Gd) {
    // A CTA without work.  The two-per-SM form always launches one CTA per SM, so that every SM holds exactly
    // one CTA of this launch and one of the next (two CTAs of one launch on an SM halve each other's speed,
    // and the launch ends with the slower ones).  A spare CTA therefore keeps its place for about as long as
    // the working ones: until the first of them says that it has begun its last round of units.  The word
    // they count up is never reset (what matters is that it changes), and the wait is bounded.
    pdl_launch_dependents();
    if (threadIdx.x != 0) return;
    pdl_wait();                                  // the earlier launch is complete: its count is final
    const unsigned before = *reinterpret_cast<volatile unsigned*>(sp.leave_signal);
    for (int i = 0; i < 20000; ++i) {
      __nanosleep(100);
      if (*reinterpret_cast<volatile unsigned*>(sp.leave_signal) != before) break;
    }
    return;
  }
  pdl_launch_dependents();
  const unsigned share = sp.share, per = sp.per;
  const int u0 = (int)(__umulhi((unsigned)blockIdx.x * share, sp.magic_grid) * per);
  const int u1 = (int)(__umulhi(((unsigned)blockIdx.x + 1u) * share, sp.magic_grid) * per);
  const int tile_first = (int)__umulhi((unsigned)u0, sp.magic_upt), tile_last = (int)__umulhi((unsigned)(u1 - 1), sp.magic_upt);
  const uint32_t meta_tx = (uint32_t)G * 80u;

  if (warp == W) {
    // ---- metadata, prefetches, refills -----------------------------------------------------------------
    if (lane < 2) mbar_init(&mfull[lane], 1);
    else if (lane < 4) mbar_init(&mempty[lane - 2], W);
    else if (lane == 5) mbar_init(rfull, 1);
    if (lane == 4) {
      flags[0] = 0;
      tma_prefetch_desc(&smap); tma_prefetch_desc(&zmap); tma_prefetch_desc(&pmap);
      if (sp.next_rows > 0) tma_prefetch_desc(&nmap);
    }
    if (lane < 6) mbar_fence_init();
    __syncwarp();
    // scales and zero points of all groups of a column tile: one box each into slot (tile - tile_first) & 1
    auto issue_meta = [&](int tile) {
      const int seq = tile - tile_first, slot = seq & 1;
      if (seq >= 2 && !mbar_wait_sleep_bounded(&mempty[slot], ((seq >> 1) & 1) ^ 1, 200000u)) {
        flags[0] = 1; atomicExch(sp.status, Q4_STATUS_WAIT_EXPIRED);
      }
      unsigned char* m = smem + L.meta + slot * L.meta_slot;
      mbar_arrive_expect_tx(&mfull[slot], meta_tx);
      tma_load_2d(m, &smap, tile * GEMV_TN, 0, &mfull[slot]);
      tma_load_2d(m + L.meta_zp, &zmap, tile * (GEMV_TN / 8), 0, &mfull[slot]);
    };
    if (lane < 2 && tile_first + lane <= tile_last) issue_meta(tile_first + lane);     // the first two tiles: no waiting
    __syncwarp();
    auto issue_prefetches = [&]() {
      if (lane >= W) return;
      if (sp.prefetch_rows > 0) {
        // Ask for the rest of this CTA's share of the layer (what the rings do not hold yet) to be brought into
        // L2 now, in boxes of `prefetch_rows` packed rows: HBM then streams at its own pace, whatever the
        // consumers do, and the refills find their bytes a short way off instead of a DRAM round trip away.
        const int upb = sp.prefetch_rows / GEMV_UNIT_ROWS;                 // units per prefetch box
        const int bpt = (upt + upb - 1) / upb;                             // boxes per column tile
        for (int item = lane; item < (tile_last - tile_first + 1) * bpt; item += W) {
          const int tl = tile_first + item / bpt, bx = item - (item / bpt) * bpt;
          const int first_u = tl * upt + bx * upb, last_u = min(tl * upt + upt, first_u + upb) - 1;
          if (last_u >= u0 + W * S && first_u < u1) tma_prefetch_l2_2d(&pmap, tl * GEMV_TN, bx * sp.prefetch_rows);
        }
      }
      if (sp.next_rows > 0) {
        // The layer that runs after this one (q4_layer_set_next): every CTA asks for its share of that layer's
        // packed weights.  Nothing here depends on an earlier kernel: weights are never written.
        const int total = sp.next_tiles * sp.next_bpt;
        for (int item = (int)blockIdx.x * W + lane; item < total; item += Gd * W) {
          const int tl = item / sp.next_bpt, bx = item - tl * sp.next_bpt;
          tma_prefetch_l2_2d(&nmap, tl * GEMV_TN, bx * sp.next_rows);
        }
      }
    };
    // Two per SM: the prefetches go out at once.  One per SM: only after the consumers have asked for x (the
    // barrier below) - a few kilobytes that wait microseconds when they queue behind megabytes of weights.
    if (OCC == 2) issue_prefetches();
    named_bar_sync_all(4, ALL);       // the consumers' barriers exist from here on (they set them up themselves)
    if (OCC == 1) issue_prefetches();
    if (lane < W) {
      constexpr unsigned MASK = (1u << W) - 1u;
      // lane c follows consumer c: its units are u0 + c + W n; the first S of them are under way already
      int n = 0, u = u0 + lane;
      int tile = (int)__umulhi((unsigned)u, sp.magic_upt), ux = u - tile * upt;
      auto advance = [&]() { u += W; ux += W; ++n; while (ux >= upt) { ux -= upt; ++tile; } };
      for (int r = 0; r < S; ++r)
        if (u < u1) {
          if (ux == 0 && tile - tile_first >= 2) issue_meta(tile);   // a short tile that opens inside the first rounds
          advance();
        }
      bool more = u < u1;
      if (TRACE && lane == 0) trace_mark(trc, 16);
      // a stage is refilled as soon as it is released, whatever the other consumers are doing (the polls do
      // not block); the lane whose unit opens a column tile brings that tile's metadata first
      uint32_t idle = 0;
      while (__any_sync(MASK, more)) {
        const bool ready = more && mbar_test_wait(&empty[lane * S + n % S], ((n / S) & 1) ^ 1);
        if (ready) {
          if (ux == 0 && tile - tile_first >= 2) issue_meta(tile);
          const int st = n % S;
          mbar_arrive_expect_tx(&full[lane * S + st], GEMV_UNIT_BYTES);
          tma_load_2d(smem + (size_t)(lane * S + st) * GEMV_UNIT_BYTES, &wmap, tile * GEMV_TN, ux * GEMV_UNIT_ROWS, &full[lane * S + st]);
          advance();
          more = u < u1;
        }
        if (__any_sync(MASK, ready)) { idle = 0; continue; }
        __nanosleep(40);
        if (++idle > (flags[0] ? 64u : 4000000u)) {
          if (lane == 0) { flags[0] = 1; atomicExch(sp.status, Q4_STATUS_WAIT_EXPIRED); }
          break;
        }
      }
    }
    return;
  }

  // A column tile whose units are dealt to two or more CTAs: the CTA that holds its first units owns it (the tile
  // is the last of its run), the others hold its later units at the start of their runs.  They finish their
  // part first and leave its 32 sums, each with a flag in one 8-byte word, in their slot of the workspace;
  // the owner's helper warp collects them while the owner's consumers are still busy, and clears the slots.
  const bool owns_shared = u1 < (tile_last + 1) * upt && u0 <= tile_last * upt;
  if (warp == W + 1) {
    named_bar_sync_all(4, ALL);
    if (!owns_shared) return;
    pdl_wait();                                  // the workspace belongs to the stream order
    const int c_last = unit_owner((long long)tile_last * upt + upt - 1, Gd, nu);
    float acc = 0.f;
    for (int cc = (int)blockIdx.x + 1; cc <= c_last; ++cc) {
      volatile unsigned long long* slot = sp.slots + (size_t)cc * 32 + lane;
      unsigned long long v = *slot;
      for (int i = 0; (v >> 32) == 0ull && i < (flags[0] ? 8 : 100000); ++i) { __nanosleep(100); v = *slot; }
      if ((v >> 32) == 0ull) { flags[0] = 1; atomicExch(sp.status, Q4_STATUS_WAIT_EXPIRED); }
      acc += __uint_as_float((unsigned)v);       // in CTA order: the result does not depend on timing
      *slot = 0ull;
    }
    remote[lane] = acc;
    __syncwarp();
    if (lane == 0) mbar_arrive(rfull);
    return;
  }
  // ---- consumers ---------------------------------------------------------------------------------------
  if (TRACE && threadIdx.x == 0 && trc) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    trc[(size_t)blockIdx.x * 64 + 47] = smid + 1;
  }
  // own barriers, then the copies that fill the own ring: weights never depend on an earlier kernel
  if (lane < S) { mbar_init(&full[warp * S + lane], 1); mbar_init(&empty[warp * S + lane], 1); }
  if (lane < S) mbar_fence_init();
  if (warp == 0 && lane == 0) tma_prefetch_desc(&wmap);
  __syncwarp();
  // rounds [r0, r1) of this consumer's ring
  auto fill_ring = [&](int r0, int r1) {
    if (lane == 0) {
      int u = u0 + warp + W * r0;
      int tile = (int)__umulhi((unsigned)u, sp.magic_upt), ux = u - tile * upt;
#pragma unroll 1
      for (int r = r0; r < r1 && u < u1; ++r) {
        mbar_arrive_expect_tx(&full[warp * S + r], GEMV_UNIT_BYTES);
        tma_load_2d(smem + (size_t)(warp * S + r) * GEMV_UNIT_BYTES, &wmap, tile * GEMV_TN, ux * GEMV_UNIT_ROWS, &full[warp * S + r]);
        u += W; ux += W;
        while (ux >= upt) { ux -= upt; ++tile; }
      }
    }
  };
  // Two per SM: all copies go out at once, long before the earlier launch is done.  One per SM: this CTA
  // started when the earlier launch was all but over; its first round goes out at once, the rest only after
  // x has been asked for - the few kilobytes of x wait microseconds when they queue behind megabytes of weights.
  fill_ring(0, OCC == 2 ? S : 1);
  if (threadIdx.x == 0) trace_mark_ns(trc, 41);
  // x as 16-bit block fixed point, for the whole of K, by all consumers together.  CT is a multiple of 16, so
  // the 16 lanes that share a group of 128 rows always hold the 16 blocks (of 8 rows) of one group.
  pdl_wait();                                  // x belongs to the stream order
  if (threadIdx.x == 0) trace_mark_ns(trc, 42);
  {
    const int K = p.K, n_blocks = upt * 32;
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    // (every CTA of the launch reads the same few kilobytes at the same moment: each starts at a different
    //  place, a whole number of groups in, and wraps around)
    const int rot = (int)(((unsigned)blockIdx.x * 2654435761u) >> 8) % (n_blocks >> 4) * 16;
    // a thread converts up to four blocks per pass; the passes' loads are issued together
    for (int base = 0; base < n_blocks; base += 4 * CT) {
      uint4 v[4];
      int blk[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = base + i * CT + (int)threadIdx.x;
        int b = idx + rot;
        if (b >= n_blocks) b -= n_blocks;
        blk[i] = idx < n_blocks ? b : n_blocks;
        if (base + i * CT < n_blocks) v[i] = 8 * blk[i] < K ? __ldg(xg + blk[i]) : make_uint4(0u, 0u, 0u, 0u);
      }
      if (OCC == 1 && base == 0) fill_ring(1, S);        // x is on its way: now the rest of the ring
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (base + i * CT >= n_blocks) break;            // the same for the whole CTA
        const __half2 h01 = as_h2(v[i].x), h23 = as_h2(v[i].y), h45 = as_h2(v[i].z), h67 = as_h2(v[i].w);
        // largest magnitude of the group (16 lanes x 8 rows), kept as a pair of halves until the end
        __half2 m2 = __hmax2(__hmax2(__habs2(h01), __habs2(h23)), __hmax2(__habs2(h45), __habs2(h67)));
#pragma unroll
        for (int d = 8; d >= 1; d >>= 1) m2 = __hmax2(m2, as_h2(__shfl_xor_sync(0xffffffffu, as_u32(m2), d)));
        const uint32_t mb = as_u32(m2);
        uint32_t ef = max(mb & 0x7FFFu, mb >> 16) >> 10;   // exponent field of the largest: 2^(ef-15) <= amax < 2^(ef-14)
        // to_int = 2^(29 - ef) makes |x_int| < 2^15; a group of subnormals and zeros (field 0) converts like
        // field 1; an infinity or a NaN (field 31) poisons the group's scale, hence its products
        const bool bad = ef == 31u;
        ef = ef ? ef : 1u;
        const float to_int = __uint_as_float((156u - ef) << 23);
        const float from_int = bad ? __uint_as_float(0x7FC00000u) : __uint_as_float((98u + ef) << 23);
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23), f45 = __half22float2(h45), f67 = __half22float2(h67);
        // x * to_int + 1.5 * 2^23: the float's low 16 bits are x_int in two's complement (round to nearest even)
        const float magic = 12582912.f;
        const uint32_t x0 = __float_as_uint(fmaf(f01.x, to_int, magic)), x1 = __float_as_uint(fmaf(f01.y, to_int, magic));
        const uint32_t x2 = __float_as_uint(fmaf(f23.x, to_int, magic)), x3 = __float_as_uint(fmaf(f23.y, to_int, magic));
        const uint32_t x4 = __float_as_uint(fmaf(f45.x, to_int, magic)), x5 = __float_as_uint(fmaf(f45.y, to_int, magic));
        const uint32_t x6 = __float_as_uint(fmaf(f67.x, to_int, magic)), x7 = __float_as_uint(fmaf(f67.y, to_int, magic));
        // digits: bytes (lo, hi) of the 16-bit two's complement x_int; even rows and odd rows apart
        const uint32_t e02 = prmt(x0, x2, 0x5140), e46 = prmt(x4, x6, 0x5140);   // lo0 lo2 hi0 hi2
        const uint32_t o13 = prmt(x1, x3, 0x5140), o57 = prmt(x5, x7, 0x5140);
        const uint4 dg = make_uint4(prmt(e02, e46, 0x7632), prmt(o13, o57, 0x7632),      // hi even, hi odd
                                    prmt(e02, e46, 0x5410), prmt(o13, o57, 0x5410));     // lo even, lo odd
        if (blk[i] < n_blocks) *reinterpret_cast<uint4*>(xp + (size_t)blk[i] * 16) = dg;
        // sum of the eight x_int: the float patterns minus eight times the pattern of the magic number
        int xs = (int)(((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7)) - 8u * 0x4B400000u);
#pragma unroll
        for (int d = 8; d >= 1; d >>= 1) xs += __shfl_xor_sync(0xffffffffu, xs, d);
        if ((lane & 15) == 0 && blk[i] < n_blocks) xinfo[blk[i] >> 4] = make_float2(from_int, (float)xs);
      }
    }
  }
  named_bar_sync(3, CT);                          // x is converted
  named_bar_sync_all(4, ALL);                     // the metadata barriers exist
  if (threadIdx.x == 0) trace_mark_ns(trc, 43);
  const int g = lane >> 2, t = lane & 3;
  // Packed words: lane (g, t) takes columns 4g..4g+3 of rows 2t (+1) of every block of eight rows.  With the
  // rows a quarter-warp reads two apart, the swizzle puts its eight 16-byte chunks on eight different bank groups.
  const uint32_t woff0 = 128u * (2 * t) + 16u * (g ^ (2 * t)), woff1 = 128u * (2 * t + 1) + 16u * (g ^ (2 * t + 1));
  float yacc[4] = {0.f, 0.f, 0.f, 0.f};                              // lanes t = 0: columns 4g .. 4g+3 of the row
  float ycorr = 0.f;                                                 // lane = column: zero points
  const unsigned char* my_stages = smem + (size_t)warp * S * GEMV_UNIT_BYTES;

  auto finish_tile = [&](int tile, int seq, int seg_first, int seg_last) {
    const bool reducer = warp == W - 1;
    if (!reducer && seq >= 1) named_bar_sync(2, CT);
    float* mine = red + warp * GEMV_TN;
    if (t == 0) *reinterpret_cast<float4*>(mine + 4 * g) = make_float4(yacc[0], yacc[1], yacc[2], yacc[3]);
    yacc[0] = yacc[1] = yacc[2] = yacc[3] = 0.f;
    __syncwarp();
    mine[lane] -= ycorr;
    ycorr = 0.f;
    if (!reducer) {
      __threadfence_block();
      named_bar_arrive(1, CT);
      return;
    }
    named_bar_sync(1, CT);
    const int tc0 = tile * GEMV_TN, col = lane;
    const bool whole = seg_first == 0 && seg_last == upt - 1;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) v += red[w * GEMV_TN + col];
    named_bar_arrive(2, CT);
    if (whole) { store_y(p, 0, tc0 + col, v); return; }
    if (seg_first > 0) {
      // a later part of a tile another CTA owns: sum and flag in one 8-byte store (one store is atomic, so
      // the owner never sees a flag without its sum, and nothing has to be fenced)
      sp.slots[(size_t)blockIdx.x * 32 + col] = (1ull << 32) | (unsigned long long)__float_as_uint(v);
      return;
    }
    // the first part of a tile that later CTAs continue: their sums, collected by the helper warp
    if (!mbar_spin_bounded(rfull, 0, flags[0] ? 64u : 20000000u)) { flags[0] = 1; atomicExch(sp.status, Q4_STATUS_WAIT_EXPIRED); }
    store_y(p, 0, tc0 + col, v + remote[col]);
  };

  int n = 0;
  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int seq = tile - tile_first, slot = seq & 1;
    const int seg_u1 = min(u1, (tile + 1) * upt);
    const unsigned char* meta = smem + L.meta + slot * L.meta_slot;
    bool meta_ready = false;
    for (int u = u0 + warp + W * n; u < seg_u1; ++n, u += W) {
      const int ux = u - tile * upt;
      const int st = n % S;
      const uint32_t lim = flags[0] ? 64u : 20000000u;
      if ((!meta_ready && !mbar_spin_bounded(&mfull[slot], (seq >> 1) & 1, lim)) || !mbar_spin_bounded(&full[warp * S + st], (n / S) & 1, lim)) {
        flags[0] = 1; atomicExch(sp.status, Q4_STATUS_WAIT_EXPIRED);
      }
      meta_ready = true;
      if (tile == tile_last && u + W >= seg_u1 && warp == 0 && lane == 0 && Gd < (int)gridDim.x)
        atomicAdd(sp.leave_signal, 1u);          // last round of this CTA: the spare CTAs may go (see the top)
      if (warp == 0 && lane == 0 && n < 8) trace_mark(trc, 20 + 2 * n);
      const unsigned char* wst = my_stages + (size_t)st * GEMV_UNIT_BYTES;
      const uint4* xq = reinterpret_cast<const uint4*>(xp + 512 * ux) + 2 * t;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4 wv[4], xv[4];
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
          // step (h, uu) takes packed rows 8 j + 2 t + pp of the unit, j = 2 h + uu / 2, pp = uu & 1
          wv[uu] = *reinterpret_cast<const uint4*>(wst + ((uu & 1) ? woff1 : woff0) + 1024 * (2 * h + (uu >> 1)));
          xv[uu] = xq[8 * (2 * h + (uu >> 1)) + (uu & 1)];
        }
        int chi[2][4], clo[2][4];                      // [column pair][fragment]
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
          const uint32_t w[4] = {wv[uu].x, wv[uu].y, wv[uu].z, wv[uu].w};
          uint32_t ev[4], od[4];                       // levels 0,2,4,6 and 1,3,5,7 of a word's eight rows, one per byte
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            ev[q] = w[q] & 0x0F0F0F0Fu;
            od[q] = (w[q] >> 4) & 0x0F0F0F0Fu;
          }
          if (uu == 0) {
            imma_u8s8_first(chi[0], ev[0], ev[1], od[0], od[1], xv[uu].x, xv[uu].y);
            imma_u8u8_first(clo[0], ev[0], ev[1], od[0], od[1], xv[uu].z, xv[uu].w);
            imma_u8s8_first(chi[1], ev[2], ev[3], od[2], od[3], xv[uu].x, xv[uu].y);
            imma_u8u8_first(clo[1], ev[2], ev[3], od[2], od[3], xv[uu].z, xv[uu].w);
          } else {
            imma_u8s8(chi[0], ev[0], ev[1], od[0], od[1], xv[uu].x, xv[uu].y);
            imma_u8u8(clo[0], ev[0], ev[1], od[0], od[1], xv[uu].z, xv[uu].w);
            imma_u8s8(chi[1], ev[2], ev[3], od[2], od[3], xv[uu].x, xv[uu].y);
            imma_u8u8(clo[1], ev[2], ev[3], od[2], od[3], xv[uu].z, xv[uu].w);
          }
        }
        // close the group of this half: the integer sums of the row (fragments 0 and 2: output columns of
        // the pair, batch row 0) times scale and 2^(E-14); one lane per column takes the zero point out:
        // y -= s * (z + 1) * 2^(E-14) * sum of x_int
        const int grp = 2 * ux + h;
        const float2 xi = xinfo[grp];
        const uint2 sc = *reinterpret_cast<const uint2*>(meta + grp * 64 + 8 * g);
        const float2 s01 = __half22float2(as_h2(sc.x)), s23 = __half22float2(as_h2(sc.y));
        yacc[0] = fmaf(s01.x * xi.x, (float)(chi[0][0] * 256 + clo[0][0]), yacc[0]);
        yacc[1] = fmaf(s01.y * xi.x, (float)(chi[0][2] * 256 + clo[0][2]), yacc[1]);
        yacc[2] = fmaf(s23.x * xi.x, (float)(chi[1][0] * 256 + clo[1][0]), yacc[2]);
        yacc[3] = fmaf(s23.y * xi.x, (float)(chi[1][2] * 256 + clo[1][2]), yacc[3]);
        const float sl = __half2float(*reinterpret_cast<const __half*>(meta + grp * 64 + 2 * lane));
        const uint32_t zw = *reinterpret_cast<const uint32_t*>(meta + L.meta_zp + grp * 16 + 4 * (lane >> 3));
        const float z1 = (float)(((zw >> (4 * (lane & 7))) & 0xFu) + 1u);
        ycorr = fmaf(sl * xi.x, z1 * xi.y, ycorr);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // our reads before the next TMA write
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[warp * S + st]);
      if (warp == 0 && lane == 0 && n < 8) trace_mark(trc, 21 + 2 * n);
    }
    // done with this tile's metadata (whether or not this warp had a unit in it)
    if (lane == 0) mbar_arrive(&mempty[slot]);
    if (warp == W - 1 && lane == 0 && tile == tile_last) trace_mark_ns(trc, 44);
    finish_tile(tile, seq, max(u0, tile * upt) - tile * upt, seg_u1 - 1 - tile * upt);
    if (warp == W - 1 && lane == 0 && tile == tile_last) trace_mark_ns(trc, 45);
  }
}

// ---- 2..16 rows, groups of 128: int8 MMAs fed by a conversion pass -----------------------------------------
// The lean kernel re-lays x out per 4 KiB unit, which with eight rows costs twice the instructions of the
// product itself.  Here x is converted once per call, by a small kernel of its own, into the 16-bit block
// fixed point of the one-row kernel above (digits in MMA order, 16 bytes per 8 k and row, the rows of a block
// 16 bytes apart and the blocks an odd number of 16-byte units apart, so that the eight rows and four blocks a
// quarter-warp reads fall on different banks), and the product kernel brings the digits of a round of its eight
// consumer warps with bulk copies: one chunk of 2048 k per round for up to 8 rows, two chunks of 1024 k (one
// per four warps, three slots in shared memory) for 9..16 rows, whose digits are twice as many.  Every CTA
// takes whole column tiles; within a tile unit r*8 + w goes to warp w in round r, so the warps of a round
// share the round's slice of x.  With 16 rows every weight fragment feeds two MMAs per digit (rows 0..7 and
// 8..15).  Zero points leave as integers: (sum of q x_int) - (z + 1) (sum of x_int).
constexpr int RW_W = 8, RW_S = 2;
template <int MR> struct RwCfg {
  static constexpr int PITCH = (MR + 1) * 16;           // bytes per block of 8 k: MR rows + 16 bytes of padding
  static constexpr int CH = MR / 8;                     // chunks of digits per round
  static constexpr int WC = RW_W / CH;                  // consumer warps that share a chunk
  static constexpr int XS = MR == 8 ? 2 : 3;            // chunk slots in shared memory
  static constexpr int CHUNK_BLOCKS = WC * 32;
  static constexpr int CHUNK_BYTES = CHUNK_BLOCKS * PITCH;   // 36864 (8 rows), 34816 (16 rows)
};

// x fp16 [M, K] -> digits [blocks][MR + 1][16 bytes] and per (group, row) the pair (2^(E-14), sum of x_int as int bits)
template <int MR>
__global__ void __launch_bounds__(256)
x_convert_kernel(const __half* __restrict__ x, unsigned char* __restrict__ xq, uint2* __restrict__ xinfo, int M, int K, int n_blocks) {
  pdl_launch_dependents();
  pdl_wait();                                    // x belongs to the stream order
  const int lane = threadIdx.x & 31;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;      // row-major over (row, block): 16 lanes share a row's group
  if (idx >= MR * n_blocks) return;
  const int m = idx / n_blocks, blk = idx - m * n_blocks;
  const bool live = m < M && 8 * blk < K;
  const uint4 v = live ? __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K) + blk) : make_uint4(0u, 0u, 0u, 0u);
  const __half2 h01 = as_h2(v.x), h23 = as_h2(v.y), h45 = as_h2(v.z), h67 = as_h2(v.w);
  __half2 m2 = __hmax2(__hmax2(__habs2(h01), __habs2(h23)), __hmax2(__habs2(h45), __habs2(h67)));
#pragma unroll
  for (int d = 8; d >= 1; d >>= 1) m2 = __hmax2(m2, as_h2(__shfl_xor_sync(0xffffffffu, as_u32(m2), d)));
  const uint32_t mb = as_u32(m2);
  uint32_t ef = max(mb & 0x7FFFu, mb >> 16) >> 10;
  const bool bad = ef == 31u;
  ef = ef ? ef : 1u;
  const float to_int = __uint_as_float((156u - ef) << 23);
  const float from_int = bad ? __uint_as_float(0x7FC00000u) : __uint_as_float((98u + ef) << 23);
  const float2 f01 = __half22float2(h01), f23 = __half22float2(h23), f45 = __half22float2(h45), f67 = __half22float2(h67);
  const float magic = 12582912.f;
  const uint32_t x0 = __float_as_uint(fmaf(f01.x, to_int, magic)), x1 = __float_as_uint(fmaf(f01.y, to_int, magic));
  const uint32_t x2 = __float_as_uint(fmaf(f23.x, to_int, magic)), x3 = __float_as_uint(fmaf(f23.y, to_int, magic));
  const uint32_t x4 = __float_as_uint(fmaf(f45.x, to_int, magic)), x5 = __float_as_uint(fmaf(f45.y, to_int, magic));
  const uint32_t x6 = __float_as_uint(fmaf(f67.x, to_int, magic)), x7 = __float_as_uint(fmaf(f67.y, to_int, magic));
  const uint32_t e02 = prmt(x0, x2, 0x5140), e46 = prmt(x4, x6, 0x5140), o13 = prmt(x1, x3, 0x5140), o57 = prmt(x5, x7, 0x5140);
  *reinterpret_cast<uint4*>(xq + ((size_t)blk * (MR + 1) + m) * 16) =
      make_uint4(prmt(e02, e46, 0x7632), prmt(o13, o57, 0x7632), prmt(e02, e46, 0x5410), prmt(o13, o57, 0x5410));
  int xs = (int)(((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7)) - 8u * 0x4B400000u);
#pragma unroll
  for (int d = 8; d >= 1; d >>= 1) xs += __shfl_xor_sync(0xffffffffu, xs, d);
  if ((lane & 15) == 0) xinfo[(size_t)(blk >> 4) * MR + m] = make_uint2(__float_as_uint(from_int), (uint32_t)xs);
}

struct RowsParams {
  GemvParams g;
  int upt, n_groups, tiles, n_blocks;             // units per tile, groups, column tiles, blocks of 8 k (padded to units)
  unsigned* status;
  const unsigned char* xq;                        // digits, see x_convert_kernel
  const uint2* xinfo;                             // [groups][MR]
};

struct RwLayout { int xring, xinfo, meta, meta_slot, meta_zp, red, bars, total; };
template <int MR>
__host__ __device__ inline RwLayout rw_layout(int G) {
  RwLayout l;
  l.xring = RW_W * RW_S * GEMV_UNIT_BYTES;
  l.xinfo = l.xring + RwCfg<MR>::XS * RwCfg<MR>::CHUNK_BYTES;
  l.meta = (l.xinfo + G * MR * 8 + 127) / 128 * 128;
  l.meta_zp = (G * 64 + 127) / 128 * 128;
  l.meta_slot = l.meta_zp + (G * 16 + 127) / 128 * 128;
  l.red = l.meta + 2 * l.meta_slot;
  l.bars = l.red + RW_W * MR * GEMV_TN * 4;
  l.total = l.bars + 8 * (2 * RW_W * RW_S + 11) + 16;
  return l;
}

// untiled bulk copy global -> shared, completion counted on `bar` (addresses and size multiples of 16 bytes)
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int MR>
__global__ void __launch_bounds__((RW_W + 1) * 32, 1)
gemv_rows_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                 const __grid_constant__ CUtensorMap zmap, const RowsParams rp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  using C = RwCfg<MR>;
  constexpr int W = RW_W, S = RW_S, CT = W * 32, RH = MR / 8;
  const GemvParams& p = rp.g;
  const int upt = rp.upt, G = rp.n_groups;
  const RwLayout L = rw_layout<MR>(G);
  unsigned char* xring = smem + L.xring;
  const uint2* xinfo_s = reinterpret_cast<const uint2*>(smem + L.xinfo);
  float* red = reinterpret_cast<float*>(smem + L.red);               // [W][MR][32]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);       // [W][S]
  uint64_t* empty = full + W * S;                                    // [W][S]
  uint64_t* mfull = empty + W * S;                                   // [2]
  uint64_t* mempty = mfull + 2;                                      // [2]
  uint64_t* xfull = mempty + 2;                                      // [3] the digits of a chunk have landed
  uint64_t* xempty = xfull + 3;                                      // [3] the chunk's consumers are done with them
  uint64_t* ifull = xempty + 3;                                      // [1] the (scale, sum) table has landed
  volatile int* flags = reinterpret_cast<volatile int*>(ifull + 1);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = (int)((long long)blockIdx.x * rp.tiles / gridDim.x), t1 = (int)((long long)(blockIdx.x + 1) * rp.tiles / gridDim.x);
  const int rounds = (upt + W - 1) / W;                              // rounds per column tile
  const uint32_t meta_tx = (uint32_t)G * 80u;

  if (threadIdx.x < 2 * W * S) mbar_init(&full[threadIdx.x], 1);
  else if (threadIdx.x < 2 * W * S + 2) mbar_init(&full[threadIdx.x], 1);                 // mfull
  else if (threadIdx.x < 2 * W * S + 4) mbar_init(&full[threadIdx.x], W);                 // mempty
  else if (threadIdx.x < 2 * W * S + 7) mbar_init(&full[threadIdx.x], 1);                 // xfull
  else if (threadIdx.x < 2 * W * S + 10) mbar_init(&full[threadIdx.x], C::WC);            // xempty
  else if (threadIdx.x == 2 * W * S + 10) mbar_init(ifull, 1);
  if (threadIdx.x == 2 * W * S + 11) {
    flags[0] = 0;
    tma_prefetch_desc(&wmap); tma_prefetch_desc(&smap); tma_prefetch_desc(&zmap);
  }
  if (threadIdx.x < 2 * W * S + 11) mbar_fence_init();
  __syncthreads();
  pdl_launch_dependents();
  auto expired = [&]() { flags[0] = 1; atomicExch(rp.status, Q4_STATUS_WAIT_EXPIRED); };

  if (warp == W) {
    // ---- issuer: lane w the units of consumer w, lane W the rounds' digits, lane W + 1 the tiles' metadata ----
    int n = 0;                                   // units issued for this lane's consumer
    int rc = 0;                                  // rounds issued (all tiles)
    int xq_next = 0;                             // chunks of digits issued (lane W): chunk q = round q / CH of the CTA, part q % CH
    bool waited = false;
    const int total_rounds = (t1 - t0) * rounds;
    const int first_rounds = total_rounds < S ? total_rounds : S;   // rounds whose weights go out before the wait
    // chunk q of the CTA: blocks [(q / CH % rounds) * W * 32 + (q % CH) * CHUNK_BLOCKS, + CHUNK_BLOCKS) of the digits
    auto issue_chunk = [&](int q) {
      const int slot = q % C::XS;
      if (q >= C::XS && !mbar_wait_sleep_bounded(&xempty[slot], ((q / C::XS) & 1) ^ 1, flags[0] ? 4u : 200000u)) expired();
      const int b0 = ((q / C::CH) % rounds) * (W * 32) + (q % C::CH) * C::CHUNK_BLOCKS;
      const int blocks = min(C::CHUNK_BLOCKS, rp.n_blocks - b0);
      mbar_arrive_expect_tx(&xfull[slot], blocks > 0 ? (uint32_t)blocks * C::PITCH : 0u);
      if (blocks > 0) bulk_load(xring + slot * C::CHUNK_BYTES, rp.xq + (size_t)b0 * C::PITCH, (uint32_t)blocks * C::PITCH, &xfull[slot]);
    };
    for (int tile = t0; tile < t1; ++tile) {
      const int seq = tile - t0, mslot = seq & 1;
      if (lane == W + 1) {
        if (seq >= 2 && !mbar_wait_sleep_bounded(&mempty[mslot], ((seq >> 1) & 1) ^ 1, 200000u)) expired();
        unsigned char* m = smem + L.meta + mslot * L.meta_slot;
        mbar_arrive_expect_tx(&mfull[mslot], meta_tx);
        tma_load_2d(m, &smap, tile * GEMV_TN, 0, &mfull[mslot]);
        tma_load_2d(m + L.meta_zp, &zmap, tile * (GEMV_TN / 8), 0, &mfull[mslot]);
      }
      for (int r = 0; r < rounds; ++r, ++rc) {
        const int ux = r * W + lane;
        if (lane < W && ux < upt) {              // weights never depend on an earlier kernel: they go first
          const int st = n % S;
          if (n >= S && !mbar_wait_sleep_bounded(&empty[lane * S + st], ((n / S) & 1) ^ 1, flags[0] ? 4u : 200000u)) expired();
          mbar_arrive_expect_tx(&full[lane * S + st], GEMV_UNIT_BYTES);
          tma_load_2d(smem + (size_t)(lane * S + st) * GEMV_UNIT_BYTES, &wmap, tile * GEMV_TN, ux * GEMV_UNIT_ROWS, &full[lane * S + st]);
          ++n;
        }
        if (!waited && rc + 1 >= first_rounds) { // the rings are filling: now the digits, which the conversion kernel writes
          __syncwarp();
          pdl_wait();
          waited = true;
          if (lane == W) {
            mbar_arrive_expect_tx(ifull, (uint32_t)G * MR * 8u);
            bulk_load(smem + L.xinfo, rp.xinfo, (uint32_t)G * MR * 8u, ifull);
          }
        }
        if (waited && lane == W)                 // the digits of every round passed so far
          for (; xq_next < (rc + 1) * C::CH; ++xq_next) issue_chunk(xq_next);
        __syncwarp();
      }
    }
    if (!waited) pdl_wait();
    return;
  }

  // ---- consumers ---------------------------------------------------------------------------------------------
  pdl_wait();                                    // y belongs to the stream order
  const int g = lane >> 2, t = lane & 3;
  const uint32_t woff0 = 128u * (2 * t) + 16u * (g ^ (2 * t)), woff1 = 128u * (2 * t + 1) + 16u * (g ^ (2 * t + 1));
  const unsigned char* my_stages = smem + (size_t)warp * S * GEMV_UNIT_BYTES;
  float yacc[RH][2][4];                          // [row half][column pair][fragment]: columns 4g + 2 cp + (i >> 1), rows 8 rh + 2t + (i & 1)
#pragma unroll
  for (int rh = 0; rh < RH; ++rh)
#pragma unroll
    for (int cp = 0; cp < 2; ++cp)
#pragma unroll
      for (int i = 0; i < 4; ++i) yacc[rh][cp][i] = 0.f;
  const uint32_t lim0 = 20000000u;
  if (!mbar_spin_bounded(ifull, 0, lim0)) expired();
  const int part = warp / C::WC, wc = warp % C::WC;

  int n = 0, rc = 0;
  for (int tile = t0; tile < t1; ++tile) {
    const int seq = tile - t0, mslot = seq & 1;
    const unsigned char* meta = smem + L.meta + mslot * L.meta_slot;
    if (!mbar_spin_bounded(&mfull[mslot], (seq >> 1) & 1, flags[0] ? 64u : lim0)) expired();
    for (int r = 0; r < rounds; ++r, ++rc) {
      const int q = rc * C::CH + part, xs = q % C::XS, ux = r * W + warp;
      if (!mbar_spin_bounded(&xfull[xs], (q / C::XS) & 1, flags[0] ? 64u : lim0)) expired();
      if (ux < upt) {
        const int st = n % S;
        if (!mbar_spin_bounded(&full[warp * S + st], (n / S) & 1, flags[0] ? 64u : lim0)) expired();
        const unsigned char* wst = my_stages + (size_t)st * GEMV_UNIT_BYTES;
        // digits of this warp's unit: block b of the chunk at b * PITCH, row m at + 16 m
        const unsigned char* xq = xring + xs * C::CHUNK_BYTES + (size_t)(wc * 32 + 2 * t) * C::PITCH + 16 * g;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          int chi[RH][2][4], clo[RH][2][4];
#pragma unroll
          for (int uu = 0; uu < 4; ++uu) {
            const uint4 wv = *reinterpret_cast<const uint4*>(wst + ((uu & 1) ? woff1 : woff0) + 1024 * (2 * h + (uu >> 1)));
            uint4 xv[RH];
#pragma unroll
            for (int rh = 0; rh < RH; ++rh)
              xv[rh] = *reinterpret_cast<const uint4*>(xq + (size_t)(8 * (2 * h + (uu >> 1)) + (uu & 1)) * C::PITCH + 128 * rh);
            const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t ev[4], od[4];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) { ev[q4] = w[q4] & 0x0F0F0F0Fu; od[q4] = (w[q4] >> 4) & 0x0F0F0F0Fu; }
#pragma unroll
            for (int rh = 0; rh < RH; ++rh) {
              if (uu == 0) {
                imma_u8s8_first(chi[rh][0], ev[0], ev[1], od[0], od[1], xv[rh].x, xv[rh].y);
                imma_u8u8_first(clo[rh][0], ev[0], ev[1], od[0], od[1], xv[rh].z, xv[rh].w);
                imma_u8s8_first(chi[rh][1], ev[2], ev[3], od[2], od[3], xv[rh].x, xv[rh].y);
                imma_u8u8_first(clo[rh][1], ev[2], ev[3], od[2], od[3], xv[rh].z, xv[rh].w);
              } else {
                imma_u8s8(chi[rh][0], ev[0], ev[1], od[0], od[1], xv[rh].x, xv[rh].y);
                imma_u8u8(clo[rh][0], ev[0], ev[1], od[0], od[1], xv[rh].z, xv[rh].w);
                imma_u8s8(chi[rh][1], ev[2], ev[3], od[2], od[3], xv[rh].x, xv[rh].y);
                imma_u8u8(clo[rh][1], ev[2], ev[3], od[2], od[3], xv[rh].z, xv[rh].w);
              }
            }
          }
          // close the group: integer sums minus (z + 1) * sum of x_int, times scale and the row's 2^(E-14)
          const int grp = 2 * ux + h;
          const uint2 sc = *reinterpret_cast<const uint2*>(meta + grp * 64 + 8 * g);
          const float2 s01 = __half22float2(as_h2(sc.x)), s23 = __half22float2(as_h2(sc.y));
          const float s[4] = {s01.x, s01.y, s23.x, s23.y};
          const uint32_t zw = *reinterpret_cast<const uint32_t*>(meta + L.meta_zp + grp * 16 + 4 * (g >> 1)) >> (16 * (g & 1));
#pragma unroll
          for (int rh = 0; rh < RH; ++rh) {
            const uint4 inf = *reinterpret_cast<const uint4*>(xinfo_s + (size_t)grp * MR + 8 * rh + 2 * t);    // rows 8 rh + 2t, + 1
            const float xsc[2] = {__uint_as_float(inf.x), __uint_as_float(inf.z)};
            const int xsum[2] = {(int)inf.y, (int)inf.w};
#pragma unroll
            for (int cp = 0; cp < 2; ++cp)
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int col = 2 * cp + (i >> 1), row = i & 1;
                const int z1 = (int)((zw >> (4 * col)) & 0xFu) + 1;
                const int v = chi[rh][cp][i] * 256 + clo[rh][cp][i] - z1 * xsum[row];
                yacc[rh][cp][i] = fmaf(s[col] * xsc[row], (float)v, yacc[rh][cp][i]);
              }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[warp * S + st]);
        ++n;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&xempty[xs]);
    }
    if (lane == 0) mbar_arrive(&mempty[mslot]);
    // the tile's sums: every warp leaves its [MR rows][32 columns], the last warp adds them in warp order
    const bool reducer = warp == W - 1;
    if (!reducer && seq >= 1) named_bar_sync(2, CT);
    float* mine = red + warp * MR * GEMV_TN;
#pragma unroll
    for (int rh = 0; rh < RH; ++rh)
#pragma unroll
      for (int cp = 0; cp < 2; ++cp)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          mine[(8 * rh + 2 * t + (i & 1)) * GEMV_TN + 4 * g + 2 * cp + (i >> 1)] = yacc[rh][cp][i];
          yacc[rh][cp][i] = 0.f;
        }
    if (!reducer) {
      __threadfence_block();
      named_bar_arrive(1, CT);
    } else {
      named_bar_sync(1, CT);
      for (int r = 0; r < p.M; ++r) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w) v += red[(w * MR + r) * GEMV_TN + lane];
        store_y(p, r, tile * GEMV_TN + lane, v);
      }
      named_bar_arrive(2, CT);
    }
  }
}

// ---- act-order (group of row k = g_idx[k]) -------------------------------------------------------
// Scale and (z+1) of the CTA's 32 columns for every group live in shared memory as half2
// (s, z+1); every element is dequantised as s*(q - (z+1)) in fp16 pairs before the MMA.
// The four lanes that share the columns 4g..4g+3 (t = 0..3) hold different k-rows, hence different
// groups: reading one table they would meet on the same bank in different rows.  The table is
// therefore kept four times, copy t with the columns of every quad rotated by t, so that the 32
// lanes of a lookup fall on 32 different banks whatever their groups are (copies = 4; layers with so
// many groups that four copies do not fit keep one, copies = 1).
template <int MT>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_act_kernel(const GemvParams p, int G, int copies) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  float* red = reinterpret_cast<float*>(smem_raw);                              // [8][MT*8][32]
  __half2* tab = reinterpret_cast<__half2*>(smem_raw + sizeof(float) * GEMV_WARPS * MT * 8 * GEMV_TN);  // [G][4 copies][32]
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
    const __half2 e = __halves2half2(p.scales[(size_t)grp * N + c0 + col], __ushort2half_rn((unsigned short)z1));
#pragma unroll
    for (int tt = 0; tt < 4; ++tt)
      if (tt < copies) tab[(grp * copies + tt) * GEMV_TN + (col & ~3) + ((col + tt) & 3)] = e;
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
  const int tc = copies == 4 ? t : 0, tstride = copies * GEMV_TN;
  const __half2* tabt = tab + tc * GEMV_TN + 4 * g;               // this lane's copy, its quad of columns
  const int qpos[4] = {tc & 3, (tc + 1) & 3, (tc + 2) & 3, (tc + 3) & 3};   // where column 4g + q sits in that copy

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
        const uint32_t raw = and_or(w[q] >> (4 * m), 0x000F000Fu, 0x64006400u);
        const __half2 qq = __hsub2(as_h2(raw), as_h2(0x64006400u));              // (q_m, q_m+4)
        const __half2 ta = tabt[gi[m] * tstride + qpos[q]], tb = tabt[gi[m + 4] * tstride + qpos[q]];
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

// What q4_layer_gemv knows about the layer that follows (set around its call of q4_gemv, on the calling thread)
struct NextLayer { const int32_t* qweight; int K, N; };
static thread_local const NextLayer* t_next_layer = nullptr;

static unsigned long long* g_trace = nullptr;                 // set by q4_gemv_set_trace
static int g_gemv_variant = 0;                                // set by q4_gemv_set_variant

constexpr size_t GEMV_STATUS_OFFSET = 65536 - 4;            // status word: last 4 bytes of the head's first half
constexpr size_t GEMV_WS_SLOTS = 65536;                     // 256-byte exchange slots, one per CTA, zero between launches
constexpr int GEMV_WS_MAX_CTAS = 255;                       // slots that fit (the last 256 bytes hold the leave signal)
constexpr int GEMV_MAX_CTAS = 508;                            // upper bound on SMs for workspace sizing (4 slots' worth of
                                                              // room is kept for the 256 bytes ahead of the partial sums)

template <int MT, bool FAST, bool XS>
static int launch_stream(const CUtensorMap& map, const CUtensorMap& smap, const CUtensorMap& zmap,
                         const GemvStreamParams& sp, int grid, cudaStream_t st) {
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  // XS adds: 16 B of zeros, the chunk table (at most 16 KiB) and x itself; sized for the worst case so that the
  // attribute is set once
  const size_t smem = gemv_stream_smem<MT>() + (XS ? 16 + GEMV_XS_MAX_BYTES : 0);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    if (int e = check_cuda(cudaFuncSetAttribute(gemv_stream_kernel<MT, FAST, XS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                           "gemv smem attribute")) return e;
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GEMV_STREAM_THREADS);
  cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<MT, FAST, XS>, map, smap, zmap, sp), "gemv launch");
}

constexpr size_t GF_SMEM_LIMIT = 227 * 1024;
// two CTAs per SM: the SM has 228 KiB of shared memory and every resident CTA reserves 1 KiB of it
constexpr size_t GF_SMEM_LIMIT2 = (228 * 1024 - 2 * 1024) / 2;

template <int MR, bool TRACE, bool XC, bool V1, int W, int OCC>
static int launch_fast_xc(const CUtensorMap& map, const GemvStreamParams& sp, int grid, cudaStream_t st) {
  static std::atomic<bool> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  static_assert(OCC == 1 || (!XC && gf_smem_bytes<MR, W>(false) <= GF_SMEM_LIMIT2 && W * 32 * OCC <= 2048), "two CTAs must fit one SM");
  const size_t smem = gf_smem_bytes<MR, W>(XC) + (XC ? gf_xc_bytes(MR, sp.units_per_tile) : 0);
  if (dev < 0 || dev >= 64 || !attr_done[dev].load(std::memory_order_acquire)) {
    const size_t most = XC ? GF_SMEM_LIMIT : smem;       // XC: the size follows K, the attribute is set once
    if (int e = check_cuda(cudaFuncSetAttribute(gemv_fast_kernel<MR, TRACE, XC, V1, W, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most),
                           "gemv smem attribute")) return e;
    // all of the SM's configurable memory as shared memory, so that OCC CTAs of this size are resident together
    if (int e = check_cuda(cudaFuncSetAttribute(gemv_fast_kernel<MR, TRACE, XC, V1, W, OCC>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                (int)cudaSharedmemCarveoutMaxShared), "gemv carveout attribute")) return e;
    if (dev >= 0 && dev < 64) attr_done[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, gemv_fast_kernel<MR, TRACE, XC, V1, W, OCC>, map, map, map, sp), "gemv launch");
}

template <int W, int S, int OCC, bool TRACE>
static int launch_ws(const CUtensorMap& wmap, const CUtensorMap& smap, const CUtensorMap& zmap, const CUtensorMap& pmap,
                     const CUtensorMap& nmap, const GemvStreamParams& sp, int grid, cudaStream_t st) {
  static std::atomic<bool> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = 1024 + (size_t)ws_layout(W, S, sp.n_groups, sp.units_per_tile).total;
  if (dev < 0 || dev >= 64 || !attr_done[dev].load(std::memory_order_acquire)) {
    if (int e = check_cuda(cudaFuncSetAttribute(gemv_ws_kernel<W, S, OCC, TRACE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)(OCC == 1 ? GF_SMEM_LIMIT : GF_SMEM_LIMIT2)), "gemv smem attribute")) return e;
    if (int e = check_cuda(cudaFuncSetAttribute(gemv_ws_kernel<W, S, OCC, TRACE>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                (int)cudaSharedmemCarveoutMaxShared), "gemv carveout attribute")) return e;
    if (dev >= 0 && dev < 64) attr_done[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  if (OCC == 2 && grid < sm_count()) grid = sm_count();       // one CTA per SM, spare ones without work (see the kernel)
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3((W + 2) * 32);
  cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, gemv_ws_kernel<W, S, OCC, TRACE>, wmap, smap, zmap, pmap, nmap, sp), "gemv launch");
}

// warps of the one-CTA-per-SM form: 16, or 12 where the stages of 16 do not fit
template <int MR>
constexpr int gf_warps1() { return MR <= 4 ? 16 : 12; }

// x' of the whole layer per CTA when it fits beside the rings and the CTA has more than one column
// tile's worth of units to amortise it over; else every unit brings and re-lays its own slice
template <int MR, bool TRACE>
static int launch_fast(const CUtensorMap& map, const GemvStreamParams& sp, int grid, cudaStream_t st) {
  constexpr int W1 = gf_warps1<MR>();
  const int xmode = g_gemv_variant & 3;
  const bool fits = gf_smem_bytes<MR, W1>(true) + gf_xc_bytes(MR, sp.units_per_tile) <= GF_SMEM_LIMIT;
  const bool pays = (long long)sp.total_units > (long long)grid * sp.units_per_tile;
  // (measured: with one row the per-unit slice is as fast or faster at every shape tried - the re-layout
  //  is 10 % of a unit's instructions and the per-CTA pass delays the first unit; from two rows on the
  //  per-CTA pass wins 5-15 % wherever a CTA has more than one tile)
  const bool xc = xmode == 2 || (xmode == 0 && pays && MR >= 2);
  if (sp.g.v1) {
    if constexpr (!TRACE) {
      if (fits && xc) return launch_fast_xc<MR, false, true, true, W1, 1>(map, sp, grid, st);
      return launch_fast_xc<MR, false, false, true, W1, 1>(map, sp, grid, st);
    }
  }
  if (fits && xc) return launch_fast_xc<MR, TRACE, true, false, W1, 1>(map, sp, grid, st);
  if constexpr (MR == 1) {
    // one row, x per unit, 11 warps at two CTAs per SM (variant bit 8; measured slower than 16 warps at one per
    // SM: a warp of this kernel is bound by the latency of its own instruction stream, so fewer warps stream less)
    if (g_gemv_variant & 8) return launch_fast_xc<1, TRACE, false, false, 11, 2>(map, sp, grid, st);
  }
  return launch_fast_xc<MR, TRACE, false, false, W1, 1>(map, sp, grid, st);
}

}  // namespace q4

using namespace q4;

// ---- layer handle: the arguments of q4_gemv that do not change from token to token ------------
struct q4_layer {
  const int32_t* qweight;
  const void* scales;
  const int32_t* qzeros;
  int K, N, G, groupsize;
  // the layer announced to follow this one (q4_layer_set_next): copies of its fields, not the handle
  const int32_t* next_qweight;
  int next_K, next_N;
};

extern "C" int q4_layer_create(q4_layer_t** out, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                               int K, int N, int G, int groupsize) {
  if (!out) return fail(Q4_E_BADARG, "layer: null handle pointer");
  *out = nullptr;
  if (!qweight || !scales || !qzeros) return fail(Q4_E_BADARG, "layer: null pointer");
  if (K <= 0 || N <= 0 || G <= 0 || groupsize <= 0) return fail(Q4_E_BADARG, "layer: K=%d N=%d G=%d groupsize=%d", K, N, G, groupsize);
  if (K % 32 || N % 32) return fail(Q4_E_SHAPE, "layer: K=%d and N=%d must be multiples of 32", K, N);
  q4_layer* l = new (std::nothrow) q4_layer{qweight, scales, qzeros, K, N, G, groupsize, nullptr, 0, 0};
  if (!l) return fail(Q4_E_BADARG, "layer: out of host memory");
  *out = l;
  return Q4_OK;
}

extern "C" void q4_layer_destroy(q4_layer_t* layer) { delete layer; }

extern "C" int q4_layer_set_next(q4_layer_t* layer, const q4_layer_t* next) {
  if (!layer) return fail(Q4_E_BADARG, "layer: null handle");
  layer->next_qweight = next ? next->qweight : nullptr;
  layer->next_K = next ? next->K : 0;
  layer->next_N = next ? next->N : 0;
  return Q4_OK;
}

extern "C" int q4_gemv_set_trace(void* device_buffer) {
  g_trace = (unsigned long long*)device_buffer;
  return Q4_OK;
}

extern "C" int q4_gemv_set_variant(int variant) {
  if (variant < 0 || variant > 127 || (variant & 3) == 3 || (variant & 32)) return fail(Q4_E_BADARG, "gemv: variant %d is not a valid combination", variant);
  g_gemv_variant = variant;
  return Q4_OK;
}

extern "C" size_t q4_gemv_workspace_bytes(int M, int K, int N) {
  if (M <= 0 || K <= 0 || N <= 0 || K % 32 || N % 32) return 0;
  int S, sps;
  gemv_plan(K, N, S, sps);
  const size_t split = S > 1 ? (size_t)S * M * N * sizeof(float) : 0;           // act-order kernel
  const size_t stream = (size_t)(GEMV_MAX_CTAS + 4) * 2 * 16 * GEMV_TN * sizeof(float); // streaming kernels
  return GEMV_WS_HEAD + (split > stream ? split : stream);
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
    // v1 layers are served by the lean kernel (K in whole 256-row units) and by the streaming instance for
    // groups of whole 128-row halves; the reference's kernel takes K in multiples of 128 as well
    if (K % 128) return fail(Q4_E_SHAPE, "gemv: v1 layers need K to be a multiple of 128 (K=%d)", K);
    groupsize = K; G = 1;
  }
  if (act && !g_idx) return fail(Q4_E_BADARG, "gemv: act-order needs g_idx");
  if (!act && (groupsize % 32 || (size_t)G * groupsize < (size_t)K))
    return fail(Q4_E_SHAPE, "gemv: groupsize=%d must be a multiple of 32 and G*groupsize >= K", groupsize);
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(scales) || (act && !aligned16(g_idx)))
    return fail(Q4_E_ALIGN, "gemv: x/qweight/scales/g_idx must be 16-byte aligned");
  if ((K * 2) % 16) return fail(Q4_E_ALIGN, "gemv: row pitch of x must be a multiple of 16 bytes");
  const size_t need = q4_gemv_workspace_bytes(M, K, N);
  if (!workspace || workspace_bytes < need)
    return fail(Q4_E_WORKSPACE, "gemv: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  if (!aligned16(workspace)) return fail(Q4_E_ALIGN, "gemv: workspace must be 16-byte aligned");
  if ((size_t)(N / GEMV_TN) * sizeof(unsigned) > GEMV_STATUS_OFFSET)
    return fail(Q4_E_SHAPE, "gemv: N=%d has more column tiles than the workspace head holds", N);
  if (int e = check_device()) return e;

  // 2..16 rows, groups of 128, whole 256-row units, enough column tiles to give every CTA whole ones: the
  // int8-MMA kernel fed by the conversion pass, in its 8-row or its 16-row form
  if (M >= 2 && !act && !v1 && groupsize == 128 && K % 256 == 0 && G == K / 128 && G <= 256 && !(g_gemv_variant & 16) &&
      N / GEMV_TN >= 32) {
    const bool wide = M > 8;
    const int MR = wide ? 16 : 8, pitch = (MR + 1) * 16;
    const int upt = K / 256, n_blocks = upt * 32;
    const size_t xq_bytes = (size_t)n_blocks * pitch, info_bytes = (size_t)G * MR * 8;
    const size_t smem = 1024 + (size_t)(wide ? rw_layout<16>(G).total : rw_layout<8>(G).total);
    if (GEMV_WS_HEAD + xq_bytes + 256 + info_bytes <= workspace_bytes && smem <= GF_SMEM_LIMIT) {
      cudaStream_t st = (cudaStream_t)stream;
      unsigned char* xq = (unsigned char*)workspace + GEMV_WS_HEAD;
      uint2* xinfo = (uint2*)(xq + ((xq_bytes + 255) & ~(size_t)255));
      RowsParams rp;
      rp.g.x = (const __half*)x; rp.g.qw = (const uint32_t*)qweight; rp.g.y = y; rp.g.scales = (const __half*)scales;
      rp.g.qzeros = (const uint32_t*)qzeros; rp.g.g_idx = nullptr; rp.g.bias = (const __half*)bias;
      rp.g.M = M; rp.g.K = K; rp.g.N = N; rp.g.groupsize = groupsize; rp.g.part = nullptr; rp.g.counters = nullptr;
      rp.g.steps_total = K / 32; rp.g.steps_per_split = 0; rp.g.S = 1;
      rp.g.y_f32 = (y_dtype == Q4_F32); rp.g.accumulate = (flags & Q4_GEMV_ACCUMULATE) ? 1 : 0; rp.g.v1 = 0;
      rp.upt = upt; rp.n_groups = G; rp.tiles = N / GEMV_TN; rp.n_blocks = n_blocks;
      rp.status = (unsigned*)((char*)workspace + GEMV_STATUS_OFFSET);
      rp.xq = xq; rp.xinfo = xinfo;
      CUtensorMap wsw, sm2, zm2;
      if (int e = make_tmap_2d(&wsw, qweight, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)N, (uint64_t)(K / 8), (uint64_t)N * 4,
                               GEMV_TN, GEMV_UNIT_ROWS, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
      if (int e = make_tmap_2d(&sm2, scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)N, (uint64_t)G, (uint64_t)N * 2,
                               GEMV_TN, G, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
      if (!aligned16(qzeros)) return fail(Q4_E_ALIGN, "gemv: qzeros must be 16-byte aligned");
      if (int e = make_tmap_2d(&zm2, qzeros, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)(N / 8), (uint64_t)G, (uint64_t)(N / 8) * 4,
                               GEMV_TN / 8, G, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
      static std::atomic<bool> attr_done[64];
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev < 0 || dev >= 64 || !attr_done[dev].load(std::memory_order_acquire)) {
        if (int e = check_cuda(cudaFuncSetAttribute(gemv_rows_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GF_SMEM_LIMIT),
                               "gemv smem attribute")) return e;
        if (int e = check_cuda(cudaFuncSetAttribute(gemv_rows_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GF_SMEM_LIMIT),
                               "gemv smem attribute")) return e;
        if (dev >= 0 && dev < 64) attr_done[dev].store(true, std::memory_order_release);
      }
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[0].val.programmaticStreamSerializationAllowed = 1;
      cudaLaunchConfig_t c1 = {};
      c1.gridDim = dim3((MR * n_blocks + 255) / 256); c1.blockDim = dim3(256); c1.stream = st; c1.attrs = at; c1.numAttrs = 1;
      if (int e = check_cuda(wide ? cudaLaunchKernelEx(&c1, x_convert_kernel<16>, (const __half*)x, xq, xinfo, M, K, n_blocks)
                                  : cudaLaunchKernelEx(&c1, x_convert_kernel<8>, (const __half*)x, xq, xinfo, M, K, n_blocks),
                             "gemv conversion launch")) return e;
      int grid = sm_count();
      if (grid > rp.tiles) grid = rp.tiles;
      cudaLaunchConfig_t c2 = {};
      c2.gridDim = dim3(grid); c2.blockDim = dim3((RW_W + 1) * 32); c2.dynamicSmemBytes = smem; c2.stream = st; c2.attrs = at; c2.numAttrs = 1;
      return check_cuda(wide ? cudaLaunchKernelEx(&c2, gemv_rows_kernel<16>, wsw, sm2, zm2, rp)
                             : cudaLaunchKernelEx(&c2, gemv_rows_kernel<8>, wsw, sm2, zm2, rp), "gemv launch");
    }
  }

  // 9..16 rows on a layer the lean kernel takes: two launches of it (8 rows, then the rest) end sooner
  // than one launch of the general streaming kernel
  if (M > 8 && !act && (groupsize == 128 || groupsize % 256 == 0) && K % 128 == 0) {
    if (int e = q4_gemv(x, qweight, y, scales, qzeros, g_idx, bias, 8, K, N, G, groupsize, y_dtype, flags, workspace, workspace_bytes, stream))
      return e;
    const size_t ybytes = (size_t)N * (y_dtype == Q4_F32 ? 4 : 2);
    return q4_gemv((const char*)x + (size_t)8 * K * 2, qweight, (char*)y + 8 * ybytes, scales, qzeros, g_idx, bias, M - 8, K, N, G,
                   groupsize, y_dtype, flags, workspace, workspace_bytes, stream);
  }

  GemvParams p;
  p.x = (const __half*)x; p.qw = (const uint32_t*)qweight; p.y = y; p.scales = (const __half*)scales;
  p.qzeros = (const uint32_t*)qzeros; p.g_idx = g_idx; p.bias = (const __half*)bias;
  p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
  p.steps_total = K / 32;
  gemv_plan(K, N, p.S, p.steps_per_split);
  p.y_f32 = (y_dtype == Q4_F32); p.accumulate = (flags & Q4_GEMV_ACCUMULATE) ? 1 : 0; p.v1 = v1 ? 1 : 0;
  p.counters = (unsigned*)workspace;
  p.part = (float*)((char*)workspace + GEMV_WS_HEAD);
  cudaStream_t st = (cudaStream_t)stream;
  const int MT = M <= 8 ? 1 : 2;

  if (!act) {
    GemvStreamParams sp;
    sp.g = p;
    sp.steps_per_tile = K / 32;
    sp.units_per_tile = (K / 8 + GEMV_UNIT_ROWS - 1) / GEMV_UNIT_ROWS;
    sp.total_units = sp.units_per_tile * (N / GEMV_TN);
    sp.cta_part = p.part;
    sp.status = (unsigned*)((char*)workspace + GEMV_STATUS_OFFSET);
    sp.trace = g_trace;
    sp.group_shift = -1;
    for (int sh = 0; sh < 20; ++sh) if ((groupsize >> 5) == (1 << sh)) sp.group_shift = sh;
    int grid = sm_count();
    if (grid > GEMV_MAX_CTAS) grid = GEMV_MAX_CTAS;
    if (grid > sp.total_units) grid = sp.total_units;
    // Lean kernel: an even share of all units per CTA makes column tiles straddle CTAs, and the sums
    // of a straddled tile meet through global memory (a fence, an atomic and a read back to back at
    // the end of the CTA: measured 3 to 4 us per launch, as long as a CTA takes for 40 units).  Dealing
    // whole tiles avoids that at the price of an uneven load; take whichever ends sooner.
    sp.whole_tiles = 0;
    sp.n_groups = G;
    {
      const int tiles = N / GEMV_TN;
      const long long cost_split = (sp.total_units + grid - 1) / grid + 40;
      const int g2 = grid < tiles ? grid : tiles;
      const long long cost_whole = (long long)((tiles + g2 - 1) / g2) * sp.units_per_tile;
      if (cost_whole <= cost_split) sp.whole_tiles = 1;
      if (g_gemv_variant & 4) sp.whole_tiles = 0;         // tests and measurements: always the even split
    }
    // One row, groups of 128, whole 256-row units: the warp-specialised kernel where its tables fit.  Its CTAs
    // exchange the sums of a straddled tile through 8-byte (sum, flag) words that nobody waits for in the
    // common case, but the exchange still ends about one round of units after the last unit: measured on the
    // LLaMA-7B shapes an even split loses to whole tiles (16 warps take a tile's units in rounds of 16, and the
    // number of rounds is the same either way), so the rule above decides for this kernel as well.
    const bool ws_ok = M == 1 && !v1 && groupsize == 128 && K % 256 == 0 && G == K / 128 && G <= 256 &&
                       sp.units_per_tile <= WS_MAX_UNITS_PER_TILE && !(g_gemv_variant & 16);
    if (ws_ok && grid > GEMV_WS_MAX_CTAS) grid = GEMV_WS_MAX_CTAS;
    bool lean_ok = (long long)sp.total_units * grid < (1ll << 32);
    // group rows one unit (256 k-rows) can touch, counting a straddled group at either end
    sp.meta_rows = v1 ? 1 : (GEMV_UNIT_ROWS * 8 + groupsize - 1) / groupsize + ((GEMV_UNIT_ROWS * 8) % groupsize ? 1 : 0);
    if (sp.meta_rows > GEMV_META_ROWS) return fail(Q4_E_SHAPE, "gemv: groupsize=%d too small", groupsize);
    if (!aligned16(qzeros)) return fail(Q4_E_ALIGN, "gemv: qzeros must be 16-byte aligned");
    CUtensorMap map, smap, zmap;
    // the lean kernel divides by the grid size and by the units per tile with 32-bit multipliers: both
    // divisors at least 2 and the dividends small enough for the multiply to be exact
    // (a layer with so many units that an even split would overflow them is dealt by whole tiles)
    if (!sp.whole_tiles && (unsigned long long)sp.total_units * grid * grid >= (1ull << 32) && N / GEMV_TN >= grid) sp.whole_tiles = 1;
    const int lean_grid = sp.whole_tiles && grid > N / GEMV_TN ? N / GEMV_TN : grid;
    sp.share = sp.whole_tiles ? (unsigned)(N / GEMV_TN) : (unsigned)sp.total_units;
    sp.per = sp.whole_tiles ? (unsigned)sp.units_per_tile : 1u;
    lean_ok = lean_ok && lean_grid >= 2 && sp.units_per_tile >= 2 &&
              (unsigned long long)sp.share * lean_grid * lean_grid < (1ull << 32) &&
              ((unsigned long long)sp.total_units + 64) * sp.units_per_tile < (1ull << 32);
    if (lean_ok && M <= 8 && (groupsize == 128 || groupsize % 256 == 0) && K % 128 == 0) {
      // lean kernel: x, scales and zero points travel with the weights by 16-byte asynchronous copies,
      // so the weights are the only tensor map it uses
      grid = lean_grid;
      sp.magic_grid = (unsigned)(((1ull << 32) + grid - 1) / grid);
      sp.magic_upt = (unsigned)(((1ull << 32) + sp.units_per_tile - 1) / sp.units_per_tile);
      CUtensorMap wsw;                                    // the same boxes, chunks swizzled by the row on their way in
      if (int e = make_tmap_2d(&wsw, qweight, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)N, (uint64_t)(K / 8),
                               (uint64_t)N * 4, GEMV_TN, GEMV_UNIT_ROWS, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
      if (ws_ok && grid <= GEMV_WS_MAX_CTAS) {
        sp.work_ctas = grid;
        sp.slots = (unsigned long long*)((char*)workspace + GEMV_WS_SLOTS);
        sp.leave_signal = (unsigned*)((char*)workspace + GEMV_WS_HEAD - 4);
        CUtensorMap sm2, zm2;                             // all groups of a column tile in one box each
        if (int e = make_tmap_2d(&sm2, scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)N, (uint64_t)G, (uint64_t)N * 2,
                                 GEMV_TN, G, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
        if (int e = make_tmap_2d(&zm2, qzeros, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)(N / 8), (uint64_t)G, (uint64_t)(N / 8) * 4,
                                 GEMV_TN / 8, G, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
        // L2 prefetch boxes: 8 units (256 packed rows) of one column tile, or the whole tile where it is shorter
        CUtensorMap pm2;
        sp.prefetch_rows = (g_gemv_variant & 64) ? 0 : (K / 8 < 256 ? K / 8 : 256);
        if (int e = make_tmap_2d(&pm2, qweight, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)N, (uint64_t)(K / 8), (uint64_t)N * 4,
                                 GEMV_TN, sp.prefetch_rows ? sp.prefetch_rows : 32, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
        // the layer the caller announced as the next one (q4_layer_set_next): boxes of up to 256 packed rows
        CUtensorMap nm2 = pm2;
        sp.next_rows = sp.next_tiles = sp.next_bpt = 0;
        if (t_next_layer && t_next_layer->qweight && !(g_gemv_variant & 64)) {
          const int rows = t_next_layer->K / 8;
          sp.next_rows = rows < 256 ? rows : 256;
          sp.next_tiles = t_next_layer->N / GEMV_TN;
          sp.next_bpt = (rows + sp.next_rows - 1) / sp.next_rows;
          if (int e = make_tmap_2d(&nm2, t_next_layer->qweight, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)t_next_layer->N, (uint64_t)rows,
                                   (uint64_t)t_next_layer->N * 4, GEMV_TN, sp.next_rows, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
        }
        const bool two_per_sm = g_gemv_variant & 8;
        if (two_per_sm && 1024 + (size_t)ws_layout(8, 2, G, sp.units_per_tile).total <= GF_SMEM_LIMIT2)
          return g_trace ? launch_ws<8, 2, 2, true>(wsw, sm2, zm2, pm2, nm2, sp, grid, st) : launch_ws<8, 2, 2, false>(wsw, sm2, zm2, pm2, nm2, sp, grid, st);
        if (1024 + (size_t)ws_layout(16, 2, G, sp.units_per_tile).total <= GF_SMEM_LIMIT)
          return g_trace ? launch_ws<16, 2, 1, true>(wsw, sm2, zm2, pm2, nm2, sp, grid, st) : launch_ws<16, 2, 1, false>(wsw, sm2, zm2, pm2, nm2, sp, grid, st);
      }
      if (g_trace && M == 1 && !v1) return launch_fast<1, true>(wsw, sp, grid, st);
      return M == 1 ? launch_fast<1, false>(wsw, sp, grid, st) : M == 2 ? launch_fast<2, false>(wsw, sp, grid, st)
           : M <= 4 ? launch_fast<4, false>(wsw, sp, grid, st) : launch_fast<8, false>(wsw, sp, grid, st);
    }
    sp.whole_tiles = 0;
    if (int e = make_tmap_2d(&map, qweight, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)N, (uint64_t)(K / 8),
                             (uint64_t)N * 4, GEMV_TN, GEMV_UNIT_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
    if (int e = make_tmap_2d(&smap, scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)N, (uint64_t)G,
                             (uint64_t)N * 2, GEMV_TN, sp.meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
    if (!v1) {
      if (int e = make_tmap_2d(&zmap, qzeros, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)(N / 8), (uint64_t)G,
                               (uint64_t)(N / 8) * 4, GEMV_TN / 8, sp.meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
      sp.stage_tx = GEMV_UNIT_BYTES + sp.meta_rows * (GEMV_TN * 2 + GEMV_TN / 2);
    } else {
      if (int e = make_tmap_2d(&zmap, qzeros, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)N, 1,
                               (uint64_t)N * 2, GEMV_TN, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
      sp.stage_tx = GEMV_UNIT_BYTES + 2 * GEMV_TN * 2;
    }
    // the instance specialised for groups of whole 128-row halves (a half-filled last unit ends after its first half)
    const bool fast = (v1 || groupsize % 128 == 0) && K % 128 == 0;
    const bool xs = fast && MT == 1 && K % 128 == 0 && (size_t)M * K * 2 + (size_t)(K / 128) * 64 <= (size_t)GEMV_XS_MAX_BYTES;
    if (xs) return launch_stream<1, true, true>(map, smap, zmap, sp, grid, st);
    if (MT == 1) return fast ? launch_stream<1, true, false>(map, smap, zmap, sp, grid, st) : launch_stream<1, false, false>(map, smap, zmap, sp, grid, st);
    return fast ? launch_stream<2, true, false>(map, smap, zmap, sp, grid, st) : launch_stream<2, false, false>(map, smap, zmap, sp, grid, st);
  }

  const dim3 grid(N / GEMV_TN, p.S), block(GEMV_THREADS);
  const size_t red_bytes = sizeof(float) * GEMV_WARPS * MT * 8 * GEMV_TN;
  const int copies = red_bytes + (size_t)G * 4 * GEMV_TN * sizeof(__half2) <= 100 * 1024 ? 4 : 1;   // two CTAs per SM at least
  const size_t smem = red_bytes + (size_t)G * copies * GEMV_TN * sizeof(__half2);
  if (smem > 200 * 1024) return fail(Q4_E_SHAPE, "gemv: act-order tables for G=%d groups do not fit shared memory", G);
  if (MT == 1) {
    if (int e = check_cuda(cudaFuncSetAttribute(gemv_act_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "gemv smem attr")) return e;
    gemv_act_kernel<1><<<grid, block, smem, st>>>(p, G, copies);
  } else {
    if (int e = check_cuda(cudaFuncSetAttribute(gemv_act_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "gemv smem attr")) return e;
    gemv_act_kernel<2><<<grid, block, smem, st>>>(p, G, copies);
  }
  return check_cuda(cudaGetLastError(), "gemv launch");
}


// The decode kernels record an expired bounded wait in the last word of the workspace head (there is one
// workspace per stream, so the word lives with it and not in a device global).
extern "C" int q4_gemv_status(const void* workspace, size_t workspace_bytes, unsigned* out) {
  if (!workspace || !out) return fail(Q4_E_BADARG, "gemv_status: null pointer");
  if (workspace_bytes < GEMV_WS_HEAD) return fail(Q4_E_WORKSPACE, "gemv_status: a decode workspace has at least %zu bytes", (size_t)GEMV_WS_HEAD);
  if (int e = check_cuda(cudaDeviceSynchronize(), "gemv_status: synchronize")) return e;
  return check_cuda(cudaMemcpy(out, (const char*)workspace + GEMV_STATUS_OFFSET, sizeof(unsigned), cudaMemcpyDeviceToHost), "read decode status");
}

extern "C" int q4_layer_gemv(const q4_layer_t* l, const void* x, void* y, int M,
                             void* workspace, size_t workspace_bytes, q4_stream_t stream) {
  if (!l) return fail(Q4_E_BADARG, "layer: null handle");
  NextLayer nx{l->next_qweight, l->next_K, l->next_N};
  t_next_layer = nx.qweight ? &nx : nullptr;
  const int rc = q4_gemv(x, l->qweight, y, l->scales, l->qzeros, nullptr, nullptr, M, l->K, l->N, l->G, l->groupsize, Q4_F16, 0u,
                         workspace, workspace_bytes, stream);
  t_next_layer = nullptr;
  return rc;
}
