// tcgen05 / TMEM wrappers (inline PTX, sm_100a) and the int4 -> fp16 dequant-to-shared-memory routine
// shared by the fused GEMM kernels.
#pragma once

#include "q4_async.cuh"

namespace q4 {

// ---- tcgen05 wrappers --------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on `bar` when all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// ---- the same for a CTA pair (cta_group::2): the even CTA of the pair issues the MMA, which reads
// 128 rows of A and half of B's columns from each CTA's shared memory and writes 128 accumulator
// rows x all N columns into each CTA's TMEM.  Allocation, release and free are issued by the same
// warp index in both CTAs.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier at this shared-memory offset in BOTH CTAs of the pair when all
// tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(both) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128B swizzle: start address, leading / stride byte offsets
// (all in 16-byte units), descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor for kind::f16: D fp32, A/B fp16, A K-major, B K-major or MN-major, M x N.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- dequantisation into the swizzled operand panels ---------------------------------------------
// Pointers into shared memory stay derived from the kernel's `extern __shared__` array by plain
// pointer arithmetic, so that the compiler keeps them in the shared address space (32-bit
// addresses, STS.128 straight from the result registers).

// Byte offsets of a task's 8 rows inside its 8-row group of a [rows][128 B] panel with the 128B
// swizzle: row J at J * 128, its 16-byte chunk `chunk` at position chunk ^ J.  Constant per thread.
__device__ __forceinline__ void deq_offsets(int chunk, uint32_t (&off)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) off[j] = j * 128 + ((chunk ^ j) << 4);
}

// Dequantise row J (nibble J of each word) of 8 packed words (8 k-rows x 8 adjacent columns) and
// write its 16-byte chunk.  `rows8` points at the task's first row, `s`/`zp` are scale and
// rn(s*(z+1)) of the 8 columns (four half2 each).
template <int J, int BYTE, bool ODD>
__device__ __forceinline__ void deq_row(unsigned char* rows8, const uint32_t (&off)[8], const uint32_t (&w)[8], const uint4& s, const uint4& zp) {
  const uint32_t sv[4] = {s.x, s.y, s.z, s.w}, zv[4] = {zp.x, zp.y, zp.z, zp.w};
  uint4 o;
  uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const __half2 q = nibble_pair<BYTE, ODD>(w[2 * c], w[2 * c + 1]);
    ov[c] = as_u32(__hsub2_rn(__hmul2_rn(as_h2(sv[c]), q), as_h2(zv[c])));
  }
  *reinterpret_cast<uint4*>(rows8 + off[J]) = o;
}

// Row J with the removal of the exponent offset folded into the scaling: the level sits in the mantissa of
// 1024 + q (low nibble, ulp 1) or of 64 + q (high nibble in place, ulp 1/16: exponent 0x5400), and
// fma(1024 + q, s, -1024 s) = rn(s q) with its single rounding, since (1024 + q) s - 1024 s = s q exactly and
// 1024 s is exact while it does not overflow.  `ce` / `co` hold -1024 s / -64 s of the 8 columns.  One
// instruction less per half2 than deq_row, same bits for |s| < 2.
template <int J, int BYTE, bool ODD>
__device__ __forceinline__ void deq_row_fold(unsigned char* rows8, const uint32_t (&off)[8], const uint32_t (&w)[8], const uint4& s, const uint4& zp,
                                             const uint32_t (&cv)[4]) {
  const uint32_t sv[4] = {s.x, s.y, s.z, s.w}, zv[4] = {zp.x, zp.y, zp.z, zp.w};
  constexpr uint32_t sel = BYTE | ((BYTE + 4) << 8);
  uint4 o;
  uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t u = prmt(w[2 * c], w[2 * c + 1], sel);
    const uint32_t v = ODD ? and_or(u, 0x00F000F0u, 0x54005400u) : and_or(u, 0x000F000Fu, 0x64006400u);
    ov[c] = as_u32(__hsub2_rn(__hfma2(as_h2(v), as_h2(sv[c]), as_h2(cv[c])), as_h2(zv[c])));
  }
  *reinterpret_cast<uint4*>(rows8 + off[J]) = o;
}

// All 8 rows with one scale / zero-term set (the rows share a quantisation group).
__device__ __forceinline__ void deq_task_uniform(unsigned char* rows8, const uint32_t (&off)[8], const uint32_t (&w)[8], const uint4& s, const uint4& zp) {
  if (((s.x | s.y | s.z | s.w) & 0x40004000u) == 0) {      // every |s| < 2 (exponent below 16; no inf or NaN): 1024 s is exact
    const uint32_t sv[4] = {s.x, s.y, s.z, s.w};
    uint32_t cv[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) cv[c] = as_u32(__hmul2_rn(as_h2(sv[c]), as_h2(0xE400E400u) /* -1024 */));
    deq_row_fold<0, 0, false>(rows8, off, w, s, zp, cv); deq_row_fold<2, 1, false>(rows8, off, w, s, zp, cv);
    deq_row_fold<4, 2, false>(rows8, off, w, s, zp, cv); deq_row_fold<6, 3, false>(rows8, off, w, s, zp, cv);
#pragma unroll
    for (int c = 0; c < 4; ++c) cv[c] = as_u32(__hmul2_rn(as_h2(sv[c]), as_h2(0xD400D400u) /* -64 */));
    deq_row_fold<1, 0, true>(rows8, off, w, s, zp, cv); deq_row_fold<3, 1, true>(rows8, off, w, s, zp, cv);
    deq_row_fold<5, 2, true>(rows8, off, w, s, zp, cv); deq_row_fold<7, 3, true>(rows8, off, w, s, zp, cv);
    return;
  }
  deq_row<0, 0, false>(rows8, off, w, s, zp); deq_row<1, 0, true>(rows8, off, w, s, zp);
  deq_row<2, 1, false>(rows8, off, w, s, zp); deq_row<3, 1, true>(rows8, off, w, s, zp);
  deq_row<4, 2, false>(rows8, off, w, s, zp); deq_row<5, 2, true>(rows8, off, w, s, zp);
  deq_row<6, 3, false>(rows8, off, w, s, zp); deq_row<7, 3, true>(rows8, off, w, s, zp);
}

__device__ __forceinline__ bool all_equal8(const int4& a, const int4& b) {
  return (((a.x ^ a.y) | (a.x ^ a.z) | (a.x ^ a.w) | (a.x ^ b.x) | (a.x ^ b.y) | (a.x ^ b.z) | (a.x ^ b.w)) == 0);
}

// rn(s * (z+1)) for 8 adjacent columns from their scales and the packed zero-point word.
__device__ __forceinline__ uint4 zero_terms(const uint4& s, uint32_t zw) {
  const uint32_t sv[4] = {s.x, s.y, s.z, s.w};
  uint4 o;
  uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    // (z | 0x6400) = 1024 + z exactly; minus 1023 gives z + 1 exactly
    const uint32_t pair = (((zw >> (8 * c)) & 0xFu) | (((zw >> (8 * c + 4)) & 0xFu) << 16)) | 0x64006400u;
    const __half2 z1 = __hsub2(as_h2(pair), as_h2(0x63FE63FEu) /* 1023 */);
    ov[c] = as_u32(__hmul2_rn(as_h2(sv[c]), z1));
  }
  return o;
}


// One dequant task (8 k-rows x 8 columns) with scales and zero terms from shared-memory tables laid
// out [group][ 128 scales | 128 rn(s*(z+1)) ] (512 bytes per group); `tab` already points at the
// task's 8 columns.  Rows of one group (always, without act-order) take the short path.
__device__ __forceinline__ void deq_task_tables(unsigned char* rows8, const uint32_t (&off)[8], const uint32_t (&w)[8], const int4& ga, const int4& gb,
                                                const unsigned char* tab) {
#define Q4_TAB(g, o) (*reinterpret_cast<const uint4*>(tab + (g) * 512 + (o)))
  // table entries are copied into registers before any row is stored: a reference into shared
  // memory would have to be re-read after every store (the compiler cannot rule out an overlap)
  if (all_equal8(ga, gb)) {
    const uint4 s = Q4_TAB(ga.x, 0), z = Q4_TAB(ga.x, 256);
    deq_task_uniform(rows8, off, w, s, z);
  } else {
    {
      const uint4 s0 = Q4_TAB(ga.x, 0), z0 = Q4_TAB(ga.x, 256), s1 = Q4_TAB(ga.y, 0), z1 = Q4_TAB(ga.y, 256);
      const uint4 s2 = Q4_TAB(ga.z, 0), z2 = Q4_TAB(ga.z, 256), s3 = Q4_TAB(ga.w, 0), z3 = Q4_TAB(ga.w, 256);
      deq_row<0, 0, false>(rows8, off, w, s0, z0); deq_row<1, 0, true>(rows8, off, w, s1, z1);
      deq_row<2, 1, false>(rows8, off, w, s2, z2); deq_row<3, 1, true>(rows8, off, w, s3, z3);
    }
    {
      const uint4 s0 = Q4_TAB(gb.x, 0), z0 = Q4_TAB(gb.x, 256), s1 = Q4_TAB(gb.y, 0), z1 = Q4_TAB(gb.y, 256);
      const uint4 s2 = Q4_TAB(gb.z, 0), z2 = Q4_TAB(gb.z, 256), s3 = Q4_TAB(gb.w, 0), z3 = Q4_TAB(gb.w, 256);
      deq_row<4, 2, false>(rows8, off, w, s0, z0); deq_row<5, 2, true>(rows8, off, w, s1, z1);
      deq_row<6, 3, false>(rows8, off, w, s2, z2); deq_row<7, 3, true>(rows8, off, w, s3, z3);
    }
  }
#undef Q4_TAB
}

// The same with scales and packed zero points read from global memory: `sc` / `qz` point at the
// task's 8 columns in group 0, `N` is the row length of the scales.
__device__ __forceinline__ void deq_task_global(unsigned char* rows8, const uint32_t (&off)[8], const uint32_t (&w)[8], const int4& ga, const int4& gb,
                                                const __half* sc, const uint32_t* qz, int N) {
  const int N8 = N >> 3;
  if (all_equal8(ga, gb)) {
    const uint4 s = __ldg(reinterpret_cast<const uint4*>(sc + (size_t)ga.x * N));
    deq_task_uniform(rows8, off, w, s, zero_terms(s, __ldg(qz + (size_t)ga.x * N8)));
  } else {
    const int gi[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
    uint4 s[8];
    uint32_t z[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j] = __ldg(reinterpret_cast<const uint4*>(sc + (size_t)gi[j] * N));
      z[j] = __ldg(qz + (size_t)gi[j] * N8);
    }
    deq_row<0, 0, false>(rows8, off, w, s[0], zero_terms(s[0], z[0])); deq_row<1, 0, true>(rows8, off, w, s[1], zero_terms(s[1], z[1]));
    deq_row<2, 1, false>(rows8, off, w, s[2], zero_terms(s[2], z[2])); deq_row<3, 1, true>(rows8, off, w, s[3], zero_terms(s[3], z[3]));
    deq_row<4, 2, false>(rows8, off, w, s[4], zero_terms(s[4], z[4])); deq_row<5, 2, true>(rows8, off, w, s[5], zero_terms(s[5], z[5]));
    deq_row<6, 3, false>(rows8, off, w, s[6], zero_terms(s[6], z[6])); deq_row<7, 3, true>(rows8, off, w, s[7], zero_terms(s[7], z[7]));
  }
}

// The same with the zero terms rn(s*(z+1)) precomputed in a [group, column] table `zp` laid out like
// the scales: two 16-byte loads per group instead of a load, eight nibble extractions and four
// multiplies.
__device__ __forceinline__ void deq_task_global_zp(unsigned char* rows8, const uint32_t (&off)[8], const uint32_t (&w)[8], const int4& ga, const int4& gb,
                                                   const __half* sc, const __half* zp, int N) {
#define Q4_S(g) __ldg(reinterpret_cast<const uint4*>(sc + (size_t)(g) * N))
#define Q4_Z(g) __ldg(reinterpret_cast<const uint4*>(zp + (size_t)(g) * N))
  if (all_equal8(ga, gb)) {
    const uint4 s = Q4_S(ga.x), z = Q4_Z(ga.x);
    deq_task_uniform(rows8, off, w, s, z);
  } else {
    {
      const uint4 s0 = Q4_S(ga.x), z0 = Q4_Z(ga.x), s1 = Q4_S(ga.y), z1 = Q4_Z(ga.y), s2 = Q4_S(ga.z), z2 = Q4_Z(ga.z), s3 = Q4_S(ga.w), z3 = Q4_Z(ga.w);
      deq_row<0, 0, false>(rows8, off, w, s0, z0); deq_row<1, 0, true>(rows8, off, w, s1, z1);
      deq_row<2, 1, false>(rows8, off, w, s2, z2); deq_row<3, 1, true>(rows8, off, w, s3, z3);
    }
    {
      const uint4 s0 = Q4_S(gb.x), z0 = Q4_Z(gb.x), s1 = Q4_S(gb.y), z1 = Q4_Z(gb.y), s2 = Q4_S(gb.z), z2 = Q4_Z(gb.z), s3 = Q4_S(gb.w), z3 = Q4_Z(gb.w);
      deq_row<4, 2, false>(rows8, off, w, s0, z0); deq_row<5, 2, true>(rows8, off, w, s1, z1);
      deq_row<6, 3, false>(rows8, off, w, s2, z2); deq_row<7, 3, true>(rows8, off, w, s3, z3);
    }
  }
#undef Q4_S
#undef Q4_Z
}

}  // namespace q4
