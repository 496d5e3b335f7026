// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the chunked
// WKV kernels use: mbarriers with bounded waits, TMA tile loads, tensor memory
// (TMEM) allocation, tcgen05.mma with shared-memory operand descriptors,
// tcgen05.ld/st, and the fences between the generic and async proxies.
//
// Operand tiles are always 64 rows x 64 bf16 (128 bytes per row) in the
// 128-byte-swizzled layout that a TMA load with CU_TENSOR_MAP_SWIZZLE_128B
// produces: the 16-byte chunk j of row i lives at chunk position j ^ (i & 7).
// Such a tile can be fed to tcgen05.mma either "K-major" (the 64 contiguous
// elements are the contraction dim) or "MN-major" (the rows are the
// contraction dim); see desc_kmajor()/desc_mnmajor().
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm100 {

constexpr int TILE_ROWS = 64;
constexpr int TILE_ROW_BYTES = 128;
constexpr int TILE_BYTES = TILE_ROWS * TILE_ROW_BYTES;  // 8 KiB

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a swizzled tile
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return static_cast<uint32_t>(row * TILE_ROW_BYTES + ((chunk ^ (row & 7)) << 4));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a
// hardware-defined time slice) and returns false; the caller records the
// failure and unwinds.  Nothing in these kernels ever spins without a bound.
// The polling loop is written in PTX: as a C loop the compiler unrolls it and
// treats the code after it as possibly divergent, which costs hundreds of
// instructions per kernel.  (Labels inside a { } block are local to it.)
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = 4000000u) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .u32 n;\n"
        "mov.u32 n, %3;\n"
        "WAIT_LOOP:\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "@p bra WAIT_DONE;\n"
        "sub.u32 n, n, 1;\n"
        "setp.ne.u32 p, n, 0;\n"
        "@p bra WAIT_LOOP;\n"
        "WAIT_DONE:\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(limit)
        : "memory");
    return ok != 0;
}
// The same, cut short when the word at `abort_flag` (shared memory) becomes non-zero:
// lets one thread that gave up end the waits of every other thread of the CTA.
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t *bar, uint32_t parity, const int *abort_flag,
                                                   uint32_t limit = 4000000u) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .u32 n, f;\n"
        "mov.u32 n, %3;\n"
        "WAIT_LOOP:\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "@p bra WAIT_DONE;\n"
        "ld.volatile.shared.u32 f, [%4];\n"
        "setp.ne.u32 q, f, 0;\n"
        "@q bra WAIT_DONE;\n"
        "sub.u32 n, n, 1;\n"
        "setp.ne.u32 p, n, 0;\n"
        "@p bra WAIT_LOOP;\n"
        "WAIT_DONE:\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(limit), "r"(smem_u32(abort_flag))
        : "memory");
    return ok != 0;
}

// ---------------------------------------------------------------------- TMA
// 3-D tiled load (coordinates: c0 innermost).  c0 * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const void *tmap, uint64_t *bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// pull the tile a later 3-D tiled load will fetch into L2
__device__ __forceinline__ void tma_prefetch_l2_3d(const void *tmap, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(tmap), "r"(c0), "r"(c1),
                 "r"(c2)
                 : "memory");
}
// untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16)
__device__ __forceinline__ void bulk_load_1d(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void *tmap, const void *smem_src, int c0, int c1,
                                             int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(tmap),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const void *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// --------------------------------------------------------------------- TMEM
// One full warp executes alloc/dealloc.  ncols: power of two, 32..512.
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------- tcgen05.mma
// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulate.
// a_mn / b_mn: operand is MN-major (contraction dim = tile rows).
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, bool a_mn, bool b_mn) {
    return (1u << 4)                         // D format: f32
           | (1u << 7)                       // A format: bf16
           | (1u << 10)                      // B format: bf16
           | ((a_mn ? 1u : 0u) << 15)        // A major
           | ((b_mn ? 1u : 0u) << 16)        // B major
           | ((uint32_t)(N >> 3) << 17)      // N / 8
           | ((uint32_t)(M >> 4) << 24);     // M / 16
}

// Shared-memory matrix descriptor of a swizzled tile (or a row/column window of
// one).  version = 1 (Blackwell), layout = SWIZZLE_128B, stride-dimension byte
// offset = 1024 (8 rows of 128 bytes); the leading-dimension offset is unused
// for a 64-element-wide tile.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)1 << 16;                        // leading byte offset (ignored), encoded 1
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
    d |= (uint64_t)1 << 46;                        // descriptor version
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
// K-major use: rows = M or N index (row0 must be a multiple of 8), contraction
// over the 64 contiguous elements; k16 selects the k-th group of 16 elements.
__device__ __forceinline__ uint64_t desc_kmajor(const void *tile, int row0, int k16) {
    return make_desc(smem_u32(tile) + row0 * TILE_ROW_BYTES + k16 * 32);
}
// MN-major use: the 64 contiguous elements = M or N index, contraction over
// rows; k16 selects rows [row0 + 16*k16, +16).  row0 must be a multiple of 8.
__device__ __forceinline__ uint64_t desc_mnmajor(const void *tile, int row0, int k16) {
    return make_desc(smem_u32(tile) + (row0 + 16 * k16) * TILE_ROW_BYTES);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// Arrive on `bar` when every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// -------------------------------------------------------------- tcgen05.ld/st
// 32 lanes x 16 consecutive fp32 columns: thread i of the warp gets lane
// (lane_base + i) where lane_base = 32 * (warp index % 4) is encoded in taddr.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float *v) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float *v) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float *v) {
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const float *v) {
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address = (lane << 16) | column
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col) {
    return base + ((uint32_t)lane << 16) + (uint32_t)col;
}

}  // namespace sm100
