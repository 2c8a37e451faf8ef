// PTX wrappers shared by the two forms of the bf16 GEMM (one CTA per tile, gemm_tcgen05.cu; a pair of CTAs per
// tile, gemm_pair.cu): mbarriers, TMA tile loads, tcgen05 fences and tensor-memory loads, shared-memory matrix
// descriptors.  Instructions that carry a .cta_group qualifier (alloc, mma, commit) live with the kernel that
// uses them: a kernel must use one value of the qualifier throughout.
#pragma once
#include "pk_common.cuh"
#include <cuda.h>
#include <cuda_bf16.h>

namespace xpk {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;
constexpr int kRasterGroup = 16;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(void *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// try_wait with a suspend-time hint: the thread may stay parked for up to `hint_ns` while the phase is incomplete
// (it is woken when the phase completes), so a polling loop around it turns far fewer times.
__device__ __forceinline__ bool mbar_try_wait_hint(void *bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, void *bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 64 bf16 (128 B),
// 8-row groups 1024 B apart; descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address      [0,14)
    d |= (uint64_t)0 << 16;                                // leading byte offset (unused here)
    d |= (uint64_t)(1024u >> 4) << 32;                     // stride byte offset [32,46)
    d |= (uint64_t)1 << 46;                                // version            [46,48)
    d |= (uint64_t)2 << 61;                                // SWIZZLE_128B       [61,64)
    return d;
}

// Tiles are numbered so that consecutive tickets cover kGroup row-blocks times all column-blocks: the
// CTAs of one wave share A and B k-blocks in L2.
template <int kGroup = kRasterGroup>
__device__ __forceinline__ void tile_coords(unsigned long long t, uint32_t m_tiles, uint32_t n_tiles,
                                            uint32_t &m_blk, uint32_t &n_blk) {
    const unsigned long long group_sz = (unsigned long long)kGroup * n_tiles;
    const uint32_t g = (uint32_t)(t / group_sz);
    const uint32_t r = (uint32_t)(t - (unsigned long long)g * group_sz);
    const uint32_t rows = min((uint32_t)kGroup, m_tiles - g * kGroup);
    m_blk = g * kGroup + r % rows;
    n_blk = r / rows;
}

// Rounds 32 fp32 accumulator values (one row, 32 consecutive columns) to bf16 and stores them as four 16-byte words.
__device__ __forceinline__ void store_row32_bf16(__nv_bfloat16 *dst_row, const uint32_t (&r)[32]) {
    uint4 *dst = reinterpret_cast<uint4 *>(dst_row);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        uint4 o;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
        __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
        __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
        __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
        o.x = *reinterpret_cast<uint32_t *>(&p0);
        o.y = *reinterpret_cast<uint32_t *>(&p1);
        o.z = *reinterpret_cast<uint32_t *>(&p2);
        o.w = *reinterpret_cast<uint32_t *>(&p3);
        dst[v] = o;
    }
}

} // namespace xpk
