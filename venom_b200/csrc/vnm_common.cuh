// Shared definitions of the venom_b200 CUDA library: format index maps, the kernel-private layout and
// thin inline-PTX wrappers for sm_100a (mbarrier, TMA, tcgen05).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace vnm {

// ------------------------------------------------------------------------------------------------
// Reference storage format (Format_sr_nm<half>, src/format/format_sr_nm.cpp of UDC-GAC/venom).
// Row r, group g (original columns g*m .. g*m+m-1), slot s in {0,1}; Ksp compressed columns.
// Closed forms of the loop nests at format_sr_nm.cpp:441-536.
// ------------------------------------------------------------------------------------------------
__host__ __device__ inline int64_t round_up_i64(int64_t x, int64_t y) { return (x + y - 1) / y * y; }

__host__ __device__ inline int64_t ksp_of(int K, int m) { return round_up_i64(round_up_i64(K, m) / m * 2, 16); }

__host__ __device__ inline int64_t values_index(int64_t r, int64_t g, int s, int64_t Ksp)
{
    return (r / 16) * 16 * Ksp + (g / 4) * 128 + ((r % 16) / 4) * 32 + (g % 4) * 8 + (r % 4) * 2 + s;
}
__host__ __device__ inline int64_t meta_index(int64_t r, int64_t g, int64_t Ksp)
{
    return (r / 32) * 16 * (Ksp / 8) + (g / 4) * 16 + (r % 32) / 2;
}
__host__ __device__ inline int meta_shift(int64_t r, int64_t g, int s)
{
    return (int)((r & 1) * 16 + (g % 4) * 4 + s * 2);
}

// ------------------------------------------------------------------------------------------------
// Kernel-private layout produced by the prepare step.
//
// The sparse operand is cut into row tiles of 128 rows and k-tiles of 64 compressed columns
// (= 32 groups = 128 gathered rows of B = four K=32 sparse MMAs).  For every (row tile, k-tile) one
// 18 KiB block holds
//   [0, 16384)      the 128 x 64 fp16 tile of compressed values as a K-major, 128-byte-swizzled shared
//                   memory image (row i at byte i*128, 16-byte chunk c stored at chunk c ^ (i % 8));
//   [16384, 18432)  the 2:4 metadata of the tile in tensor-memory order: word [lane*4 + kb] with
//                   lane = m0 + 8*k1 + 16*m2 and kb the K=32 block; the low half-word belongs to MMA row
//                   16*m2 + m0, the high half-word to MMA row 16*m2 + 8 + m0, both for logical columns
//                   kb*32 + k1*16 .. +15 (4 bits per group of four).
// MMA row i of a tile is actual row perm(i): inside every 16-row group MMA rows (w, w+8) are actual
// rows (2w, 2w+1), so that one reference metadata word (an even/odd row pair) is one tensor-memory word.
// A second array holds, per (V-block, group), the four absolute B row numbers g*m + colloc[j]
// (or K, which is out of range and reads as zeros, for padding).
// ------------------------------------------------------------------------------------------------
constexpr int TILE_M = 128;         // rows per CTA tile (UMMA M)
constexpr int KT_COMP = 64;         // compressed columns per k-tile
constexpr int KT_GROUPS = 32;       // groups per k-tile
constexpr int KT_ROWS = 128;        // gathered B rows per k-tile
constexpr int A_IMG_BYTES = TILE_M * KT_COMP * 2;   // 16384
constexpr int META_IMG_BYTES = TILE_M * 16;         // 2048
constexpr int AM_BLOCK_BYTES = A_IMG_BYTES + META_IMG_BYTES;  // 18432

__host__ __device__ inline int mma_row_to_actual(int i) { int w = i & 15; return (i & ~15) + ((w & 7) << 1) + (w >> 3); }
__host__ __device__ inline int actual_to_mma_row(int a) { int x = a & 15; return (a & ~15) + ((x & 1) << 3) + (x >> 1); }

// Tile order of the persistent kernels.  group > 0: row groups (units of one CTA tile's rows) are taken `group` at a
// time and, inside such a band, column tiles advance slowest: the CTAs that run together share `group` row groups
// of A, which can stay in L2 while the column panels of B stream past.  group < 0: the transposed order, bands of
// -group column tiles inside which row groups advance slowest: the band's B panels stay in L2 while A streams past
// (cheaper whenever A is the smaller operand).  Either way A is no longer re-read from HBM once per column tile, which
// is what "row groups fastest over the whole matrix" costs as soon as A is larger than L2.
__host__ __device__ inline void tile_coords(int tile, int row_groups, int ntiles, int group, int *rg, int *nt)
{
    if (group >= 0) {
        const int band = tile / (group * ntiles);
        const int first = band * group;
        const int size = row_groups - first < group ? row_groups - first : group;
        const int within = tile - band * group * ntiles;
        *nt = within / size;
        *rg = first + within % size;
    } else {
        const int g = -group;
        const int band = tile / (g * row_groups);
        const int first = band * g;
        const int size = ntiles - first < g ? ntiles - first : g;
        const int within = tile - band * g * row_groups;
        *rg = within / size;
        *nt = first + within % size;
    }
}

#if defined(__CUDACC__)
// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a barrier phase (try_wait may park the thread for a while before it reports
// completion; the single-thread pipeline roles spin on this instead to keep hand-offs short).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Bulk copy global -> shared (no tensor map): both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// L2 eviction-priority policies for the hinted copies below (the encodings createpolicy.fractional produces for a
// fraction of 1.0): lines loaded with EVICT_LAST are the last candidates for replacement, EVICT_FIRST the first.
constexpr uint64_t L2_EVICT_NORMAL = 0x1000000000000000ull;
constexpr uint64_t L2_EVICT_FIRST = 0x12F0000000000000ull;
constexpr uint64_t L2_EVICT_LAST = 0x14F0000000000000ull;
__device__ __forceinline__ void bulk_g2s_hint(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(void *smem_dst, const void *tmap, int col, int row, uint64_t *bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(col), "r"(row), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void tma_load_4d_hint(void *smem_dst, const void *tmap, int c0, int c1, int c2, int c3, uint64_t *bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
// Prefetches into L2 only (no shared-memory destination, no barrier): a contiguous range, or the box of a tiled load.
__device__ __forceinline__ void bulk_prefetch_l2(const void *gsrc, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const void *tmap, int col, int row)
{
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(col), "r"(row) : "memory");
}
__device__ __forceinline__ void tma_prefetch_4d(const void *tmap, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// TMA gather: four rows (r.x..r.w) of a 2-D tensor, `col` = first element of the inner box.
__device__ __forceinline__ void tma_gather4(void *smem_dst, const void *tmap, int col, int4 r, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(col), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w), "r"(smem_u32(bar))
        : "memory");
}
// TMA tile load of a 2-D box at (col, row).
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const void *tmap, int col, int row, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(col), "r"(row), "r"(smem_u32(bar))
                 : "memory");
}
// TMA tile load of a 4-D box at (c0, c1, c2, c3), c0 innermost.
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const void *tmap, int c0, int c1, int c2, int c3, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
                 : "memory");
}
// TMA tile store shared -> global of a 2-D box at (col, row); completion is tracked by bulk groups.
__device__ __forceinline__ void tma_store_2d(const void *tmap, const void *smem_src, int col, int row)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tmap), "r"(col), "r"(row),
                 "r"(smem_u32(smem_src))
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the bulk groups of this thread have finished READING shared memory (the source may be reused).
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
// Named barrier that also returns the AND of `pred` over its participants.
__device__ __forceinline__ bool named_barrier_and(uint32_t id, uint32_t threads, bool pred)
{
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.and.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(id), "r"(threads), "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}
// 8-byte asynchronous copy global -> shared (8-byte aligned on both sides), grouped with commit / wait.
__device__ __forceinline__ void cp_async_8(uint32_t saddr, const void *gsrc)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(saddr), "l"(gsrc) : "memory");
}
// 16-byte asynchronous copy global -> shared that bypasses L1; src_bytes = 16 copies, 0 writes zeros (src is not read).
__device__ __forceinline__ void cp_async_16_zfill(uint32_t saddr, const void *gsrc, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(saddr), "l"(gsrc), "r"(src_bytes) : "memory");
}
// Deferred arrival: the barrier receives one arrival (already counted in its initial count) once every asynchronous
// copy this thread has issued so far has completed.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t *bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}
// Register re-allocation between warpgroups (all four warps of a warpgroup must execute the same one).
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs)); }
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs)); }
__device__ __forceinline__ void tma_prefetch_desc(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives on `bar` once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Shared -> tensor memory copy, 128 lanes x 128 bits (four 32-bit columns).
__device__ __forceinline__ void tc_cp_128x128b(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// D[tmem] (+)= A_sparse[smem] * B[smem]; 2:4 metadata in tensor memory; `mask` disables output lanes.
__device__ __forceinline__ void tc_mma_sp_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t meta_tmem, uint32_t idesc,
                                              uint32_t accumulate, uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], %1, %2, [%3], %4, {%6, %7, %8, %9}, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(meta_tmem), "r"(idesc), "r"(accumulate), "r"(m0), "r"(m1), "r"(m2), "r"(m3)
        : "memory");
}
// Dense counterpart (used by the self-test of the descriptors).
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                           uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(m0), "r"(m1), "r"(m2), "r"(m3)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread t = lane base + t).
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of tcgen05 (64 bit): start address, leading / stride byte offsets
// (all >> 4), version 1 at bit 46, swizzle mode at bits 61-63 (0 none, 2 = 128-byte).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle_mode)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(swizzle_mode & 7) << 61;
    return d;
}
// Instruction descriptor of tcgen05.mma kind::f16 with fp16 A/B, fp32 D, A K-major, B MN-major.
//   bits 0-1 sparsity selector, 2 sparse flag, 4-5 D format (1 = f32), 7-9 A format (0 = f16),
//   10-12 B format, 15 A major (0 = K), 16 B major (1 = MN), 17-22 N >> 3, 24-28 M >> 4.
__device__ __forceinline__ uint32_t make_idesc_f16(int M, int N, bool sparse, uint32_t id2, bool b_mn_major)
{
    uint32_t d = 0;
    d |= (id2 & 3u);
    d |= (sparse ? 1u : 0u) << 2;
    d |= 1u << 4;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}
#endif  // __CUDACC__

}  // namespace vnm
