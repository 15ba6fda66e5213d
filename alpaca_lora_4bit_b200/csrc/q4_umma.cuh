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

// Dequantise 8 packed words (8 k-rows x 8 adjacent columns) and write the eight 16-byte chunks
// into a [rows][128 B] panel with the 128B swizzle.  `s`/`zp` give scale and rn(s*(z+1)) of the 8
// columns for each of the 8 rows (as four half2 each).
template <int J, int BYTE, bool ODD>
__device__ __forceinline__ void deq_row(unsigned char* panel_rows8, int chunk, const uint32_t (&w)[8],
                                        const uint4& s, const uint4& zp) {
  const uint32_t sv[4] = {s.x, s.y, s.z, s.w}, zv[4] = {zp.x, zp.y, zp.z, zp.w};
  uint4 o;
  uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const __half2 q = nibble_pair<BYTE, ODD>(w[2 * c], w[2 * c + 1]);
    ov[c] = as_u32(__hsub2_rn(__hmul2_rn(as_h2(sv[c]), q), as_h2(zv[c])));
  }
  *reinterpret_cast<uint4*>(panel_rows8 + J * 128 + ((chunk ^ J) << 4)) = o;
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


}  // namespace q4
