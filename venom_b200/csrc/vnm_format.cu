// Format kernels: dense -> V:N:M compressor + metadata packer, decompressor, and the re-pack of the
// reference-format arrays into the kernel-private layout.  All are HBM-bound byte/bit shuffles.
#include "vnm_internal.h"

namespace vnm {

// ------------------------------------------------------------------------------------------------
// Compressor, general form (any alignment, any m).  One thread owns one metadata word = (row pair 2p,2p+1) x (tile t of four groups):
// it scans 2 x 4 groups x 4 column-loc candidates of the pruned dense matrix in ascending order,
// emits the first two kept entries of every (row, group) as values + 2-bit positions, and writes one
// 32-bit metadata word plus four 8-byte value pieces.  Threads of a warp walk consecutive tiles of
// the same row pair, so the dense reads of a warp cover 32*4*m consecutive columns of two rows.
// Follows Format_sr_nm<T>::to_sparse_sr_nm (format_sr_nm.cpp:441-536): candidates with an original
// column >= K contribute a (position 0, value 0) slot for j < 2 only (:486-500).
// ------------------------------------------------------------------------------------------------
template <bool kHasMask>
__global__ void __launch_bounds__(256) compress_kernel(const __half *__restrict__ dense, int64_t ldd, const int32_t *__restrict__ mask,
                                                       const uint32_t *__restrict__ colloc, int M, int K, int V, int m, int64_t Ksp,
                                                       __half *__restrict__ values, uint32_t *__restrict__ meta,
                                                       unsigned long long *violations)
{
    const int64_t tiles = Ksp / 8;
    const int64_t total = (int64_t)(M / 2) * tiles;
    unsigned int bad = 0;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t rp = idx / tiles;
        const int64_t t = idx - rp * tiles;
        uint32_t word = 0;
        const int64_t r0 = rp * 2;
        const uint4 *c4p = reinterpret_cast<const uint4 *>(colloc + (r0 / V) * (Ksp / 2) * 4 + t * 16);
        // values of rows r0, r0+1 for group gi are 4 consecutive halves at vbase + gi*8
        const int64_t vbase = (r0 / 16) * 16 * Ksp + t * 128 + ((r0 % 16) / 4) * 32 + (r0 % 4) * 2;
#pragma unroll
        for (int gi = 0; gi < 4; gi++) {
            const uint4 c4 = __ldg(c4p + gi);
            const uint32_t cand[4] = {c4.x, c4.y, c4.z, c4.w};
            const int64_t g = t * 4 + gi;
            unsigned short out[4] = {0, 0, 0, 0};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const __half *drow = dense + (r0 + h) * ldd;
                const int32_t *mrow = kHasMask ? mask + (r0 + h) * ldd : nullptr;
                int pos = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int64_t col = g * m + (int64_t)cand[j];
                    if (cand[j] >= (uint32_t)m) {
                        pos = 3;  // a column offset outside its group (corrupt column-loc): counted as a violation, never read
                    } else if (col < K) {
                        const unsigned short bits = __half_as_ushort(drow[col]);
                        const bool keep = kHasMask ? (mrow[col] != 0) : ((bits & 0x7FFFu) != 0);  // value != +-0
                        if (keep) {
                            if (pos < 2) {
                                out[h * 2 + pos] = bits;
                                word |= (uint32_t)j << (h * 16 + gi * 4 + pos * 2);
                            }
                            pos++;
                        }
                    } else if (j < 2) {
                        pos++;  // slot (position 0, value 0): nothing to OR in
                    }
                }
                bad += (pos != 2);
            }
            uint2 pk;
            pk.x = (uint32_t)out[0] | ((uint32_t)out[1] << 16);
            pk.y = (uint32_t)out[2] | ((uint32_t)out[3] << 16);
            *reinterpret_cast<uint2 *>(values + vbase + gi * 8) = pk;
        }
        meta[(r0 / 32) * 16 * tiles + t * 16 + (r0 % 32) / 2] = word;
    }
    if (violations != nullptr) {
        for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
        if ((threadIdx.x & 31) == 0 && bad) atomicAdd(violations, (unsigned long long)bad);
    }
}

// ------------------------------------------------------------------------------------------------
// Tiled compressor (the one normally used).  A CTA takes 32 rows (inside one V-block, so one column-loc
// row) x TS tiles of four groups = TS*4*m consecutive columns:
//   1. the 32 dense row segments come in with coalesced 8-byte asynchronous copies into one of two
//      shared-memory buffers (row pitch an odd number of words, so 32 lanes reading one column of 32 rows
//      hit 32 banks), one chunk ahead of the work; in mask mode the int32 mask is folded into one bit per
//      element;
//   2. lane = row, warp = tile: the same selection as compress_kernel, results staged in shared memory in
//      the reference's value order (128 halves per 16 rows x tile) and metadata order (16 words per
//      32 rows x tile);
//   3. both stagings are contiguous in global memory (TS*256 bytes per 16 rows, TS*64 bytes of metadata)
//      and leave with 16-byte stores.
// Needs 8-byte aligned dense and mask rows and an even m; launch_compress falls back to compress_kernel
// otherwise.
// ------------------------------------------------------------------------------------------------
template <bool kHasMask>
__global__ void __launch_bounds__(256) compress_tiled_kernel(const __half *__restrict__ dense, int64_t ldd, const int32_t *__restrict__ mask,
                                                             const uint32_t *__restrict__ colloc, int M, int K, int V, int m, int64_t Ksp, int TS,
                                                             uint32_t *__restrict__ values, uint32_t *__restrict__ meta,
                                                             unsigned long long *violations)
{
    extern __shared__ __align__(16) uint8_t csm[];
    const int span = TS * 4 * m;                 // columns per chunk, even
    const int pitch = span + 4;                  // halves; 8-byte aligned rows, pitch / 2 = 2 mod 32: rows r and r+16 share banks
    const int mpitch = ((span / 2 + 7) & ~7) + 4;  // mask bytes per row (two bits per byte); mpitch / 4 is odd
    uint32_t *val_s = reinterpret_cast<uint32_t *>(csm);                 // [2][TS][64]
    uint32_t *meta_s = val_s + 2 * TS * 64;                              // [TS][16]
    unsigned short *in_s = reinterpret_cast<unsigned short *>(meta_s + TS * 16);  // [2 buffers][32][pitch]
    uint8_t *mk_s = reinterpret_cast<uint8_t *>(in_s + 2 * 32 * pitch);  // [32][mpitch]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tiles = Ksp / 8;
    const int spans = (int)((tiles + TS - 1) / TS);
    const int64_t chunks = (int64_t)(M / 32) * spans;
    unsigned int bad = 0;

    // Asynchronous 8-byte copies bring the 32 row segments of a chunk into one of two buffers: a warp takes
    // rows warp, warp+8, ..., its lanes consecutive pieces, so global reads are coalesced and shared-memory
    // writes hit consecutive banks.  The chunk after the current one is in flight while this one is worked on.
    auto fetch = [&](int64_t ch, int buf) {
        const int64_t rc = ch / spans;
        const int64_t c0 = (ch - rc * spans) * TS * 4 * m;
        const int valid = (int)(c0 >= K ? 0 : (K - c0 < span ? K - c0 : span));
        const int nq = (valid + 3) / 4;  // 8-byte pieces per row holding existing columns
        for (int r = warp; r < 32; r += 8) {
            const __half *drow = dense + (rc * 32 + r) * ldd + c0;
            unsigned short *srow = in_s + (buf * 32 + r) * pitch;
            const uint32_t sbase = smem_u32(srow);
#pragma unroll 4
            for (int q = lane; q < nq; q += 32) {
                if (4 * q + 4 <= valid) {
                    cp_async_8(sbase + q * 8, reinterpret_cast<const uint2 *>(drow) + q);
                } else {  // ragged end of the matrix
                    for (int c = 4 * q; c < valid; c++) srow[c] = __half_as_ushort(drow[c]);
                }
            }
        }
        cp_async_commit();
    };

    int buf = 0;
    if ((int64_t)blockIdx.x < chunks) fetch(blockIdx.x, 0);
    for (int64_t ch = blockIdx.x; ch < chunks; ch += gridDim.x, buf ^= 1) {
        const int64_t rc = ch / spans;
        const int sp = (int)(ch - rc * spans);
        const int64_t R0 = rc * 32;
        const int64_t t0 = (int64_t)sp * TS;
        const int tcount = (int)(tiles - t0 < TS ? tiles - t0 : TS);
        const int64_t c0 = t0 * 4 * m;
        if (ch + gridDim.x < chunks) {
            fetch(ch + gridDim.x, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        if (kHasMask) {  // the int32 mask, folded into one bit per element
            const int valid = (int)(c0 >= K ? 0 : (K - c0 < span ? K - c0 : span));
            const int nw = (valid + 1) / 2;
            for (int r = warp; r < 32; r += 8) {
                const int32_t *mrow = mask + (R0 + r) * ldd + c0;
                for (int w = lane; w < nw; w += 32) {
                    uint32_t mb;
                    if (2 * w + 1 < valid) {
                        const int2 mm = __ldg(reinterpret_cast<const int2 *>(mrow) + w);
                        mb = (mm.x != 0) | ((mm.y != 0) << 1);
                    } else {
                        mb = mrow[2 * w] != 0;
                    }
                    mk_s[r * mpitch + w] = (uint8_t)mb;
                }
            }
        }
        __syncthreads();
        // ---- lane = row, warp = tile
        const uint32_t *crow = colloc + (R0 / V) * (Ksp / 2) * 4;
        const unsigned short *my_in = in_s + (buf * 32 + lane) * pitch;
        const uint8_t *my_mk = mk_s + lane * mpitch;
        const int validc = (int)(c0 >= K ? 0 : (K - c0 < span ? K - c0 : span));
        for (int tl = warp; tl < tcount; tl += 8) {
            uint32_t hw = 0;
            uint32_t *vdst = val_s + ((lane >> 4) * TS + tl) * 64 + ((lane & 15) >> 2) * 16 + (lane & 3);
            const uint4 *c4p = reinterpret_cast<const uint4 *>(crow + (t0 + tl) * 16);
#pragma unroll
            for (int gi = 0; gi < 4; gi++) {
                const uint4 c4 = __ldg(c4p + gi);
                const int cand[4] = {(int)c4.x, (int)c4.y, (int)c4.z, (int)c4.w};
                const int lg = (tl * 4 + gi) * m;  // first column of the group, relative to the chunk
                uint32_t out = 0;
                int pos = 0;
                if (max(max(c4.x, c4.y), max(c4.z, c4.w)) >= (uint32_t)m) {
                    pos = 3;  // a column offset outside its group (corrupt column-loc): counted as a violation, nothing is read
                } else if (lg + m <= validc) {  // the whole group exists (same for every lane)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int lc = lg + cand[j];
                        const uint32_t bits = my_in[lc];
                        const bool keep = kHasMask ? ((my_mk[lc >> 1] >> (lc & 1)) & 1) != 0 : (bits & 0x7FFFu) != 0;
                        if (keep) {
                            if (pos < 2) {
                                out |= bits << (16 * pos);
                                hw |= (uint32_t)j << (gi * 4 + pos * 2);
                            }
                            pos++;
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int lc = lg + cand[j];
                        if (lc < validc) {
                            const uint32_t bits = my_in[lc];
                            const bool keep = kHasMask ? ((my_mk[lc >> 1] >> (lc & 1)) & 1) != 0 : (bits & 0x7FFFu) != 0;
                            if (keep) {
                                if (pos < 2) {
                                    out |= bits << (16 * pos);
                                    hw |= (uint32_t)j << (gi * 4 + pos * 2);
                                }
                                pos++;
                            }
                        } else if (j < 2) {
                            pos++;  // slot (position 0, value 0) of a column past K
                        }
                    }
                }
                bad += (pos != 2);
                vdst[gi * 4] = out;
            }
            const uint32_t other = __shfl_xor_sync(0xffffffffu, hw, 1);
            if ((lane & 1) == 0) meta_s[tl * 16 + (lane >> 1)] = hw | (other << 16);
        }
        __syncthreads();
        // ---- staged values and metadata -> global memory
        const int vq = tcount * 16;  // 16-byte pieces per 16-row group
        for (int i = threadIdx.x; i < 2 * vq; i += 256) {
            const int rg = i >= vq ? 1 : 0;
            const int k = i - rg * vq;
            uint4 *dst = reinterpret_cast<uint4 *>(values + ((R0 / 16 + rg) * 16 * Ksp + t0 * 128) / 2);
            dst[k] = reinterpret_cast<const uint4 *>(val_s + rg * TS * 64)[k];
        }
        uint4 *mdst = reinterpret_cast<uint4 *>(meta + (R0 / 32) * 16 * tiles + t0 * 16);
        for (int i = threadIdx.x; i < tcount * 4; i += 256) mdst[i] = reinterpret_cast<const uint4 *>(meta_s)[i];
    }
    if (violations != nullptr) {
        for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
        if (lane == 0 && bad) atomicAdd(violations, (unsigned long long)bad);
    }
}

// ------------------------------------------------------------------------------------------------
// Compressor, register form, for the common shapes: no mask, m in {4, 8, 16}, K % (4 * m) == 0 (whole tiles, no
// padded group), V a multiple of 16 and 16-byte aligned rows.  The lanes of a warp lie ALONG a row: a thread owns 16
// bytes of the row or one group, whichever is larger (two groups for m = 4, one for m = 8 and 16), so a load instruction
// of a warp reads 512 contiguous bytes (1 KiB for m = 16).  The thread walks the 16 rows of a value strip four at a
// time: for its group the kept pairs of four consecutive rows are exactly one 16-byte piece of the reference's value
// order [sub-block][group][row][slot], so it is stored straight from registers, without any exchange between lanes; the
// candidates' select predicates depend on the column-loc entry only and are shared by the 16 rows.  The lanes of a tile
// (4, or 2 for m = 4) OR their metadata nibbles together with shuffles and write the strip's 32 bytes of the tile's
// metadata as one sector.  A CTA (8 warps) covers 16 rows x 4 KiB (8 KiB for m = 16); the grid is one resident wave
// and walks the items in row-major order, so neighbouring CTAs read neighbouring pieces of the same rows.
// ------------------------------------------------------------------------------------------------
// m = 8 fits 64 registers without spilling (four CTAs per SM: measured 11 % faster than three); m = 4 and 16 do not
template <int M_>
__global__ void __launch_bounds__(256, M_ == 8 ? 4 : 1) compress_direct_kernel(const __half *__restrict__ dense, int64_t ldd, const uint32_t *__restrict__ colloc,
                                                              int V, int tiles, uint32_t spans, uint32_t items, uint32_t *__restrict__ values,
                                                              uint32_t *__restrict__ meta, unsigned long long *violations)
{
    constexpr int NW = M_ / 2;             // 32-bit words per group
    constexpr int GPT = M_ == 4 ? 2 : 1;   // groups per thread
    constexpr int TW = GPT * NW;           // words per thread and row (4, 4, 8)
    constexpr int LPR = TW / 4;            // 16-byte loads per thread and row
    constexpr int TL = 4 / GPT;            // lanes per tile
    constexpr int TPW = 32 / TL;           // tiles per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tli = lane % TL, g0 = tli * GPT;   // this thread's first group inside its tile
    const int64_t Ksp = (int64_t)tiles * 8;
    unsigned int bad = 0;
    // where the thread's 16 rows start for an item (lanes past the last tile repeat it: they take part in the shuffles)
    auto row0_of = [&](uint32_t item) {
        const uint32_t strip = item / spans;
        const int t = (int)(item - strip * spans) * (8 * TPW) + warp * TPW + lane / TL;
        const int T = t < tiles ? t : tiles - 1;
        return dense + (int64_t)strip * 16 * ldd + ((int64_t)T * 4 + g0) * M_;
    };
    auto load4 = [&](const __half *row0, int sb, uint32_t (&w)[4][TW]) {   // rows 4*sb .. 4*sb+3
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const uint4 *src = reinterpret_cast<const uint4 *>(row0 + (int64_t)(sb * 4 + r) * ldd);
#pragma unroll
            for (int i = 0; i < LPR; i++) {
                const uint4 v = __ldg(src + i);
                w[r][4 * i] = v.x; w[r][4 * i + 1] = v.y; w[r][4 * i + 2] = v.z; w[r][4 * i + 3] = v.w;
            }
        }
    };
    // The loads run one step (four rows) ahead of the arithmetic, across item boundaries: two register buffers
    uint32_t wa[4][TW], wb[4][TW];
    const __half *row0 = blockIdx.x < items ? row0_of(blockIdx.x) : dense;
    if (blockIdx.x < items) load4(row0, 0, wa);
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t strip = item / spans;
        const int t = (int)(item - strip * spans) * (8 * TPW) + warp * TPW + lane / TL;
        const bool valid = t < tiles;          // whole tiles: the lanes of a tile are valid together
        const int T = valid ? t : tiles - 1;
        const int64_t G = (int64_t)T * 4 + g0; // first group of this thread in its row
        const __half *next_row0 = item + gridDim.x < items ? row0_of(item + gridDim.x) : row0;
        // candidates of the thread's groups: the same for the 16 rows (V % 16 == 0)
        uint32_t cand[GPT][4];
        uint32_t okmask[GPT];   // 0 for a group whose column-loc entry is corrupt (an offset outside the group): every row counts a violation
        {
            const uint4 *c4p = reinterpret_cast<const uint4 *>(colloc + ((int64_t)(strip * 16u / (uint32_t)V) * (Ksp / 2) + G) * 4);
#pragma unroll
            for (int j = 0; j < GPT; j++) {
                const uint4 c4 = __ldg(c4p + j);
                const bool corrupt = max(max(c4.x, c4.y), max(c4.z, c4.w)) >= (uint32_t)M_;
                okmask[j] = corrupt ? 0u : 0xFFFFFFFFu;
                cand[j][0] = c4.x & okmask[j]; cand[j][1] = c4.y & okmask[j]; cand[j][2] = c4.z & okmask[j]; cand[j][3] = c4.w & okmask[j];
            }
        }
        uint4 *vdst = reinterpret_cast<uint4 *>(values) + ((int64_t)strip * 16 * Ksp + (int64_t)T * 128) / 8 + g0;
        uint32_t keep[4] = {0, 0, 0, 0};   // metadata words this lane stores at the end: 2 (TL = 4) or 4 (TL = 2)
        auto work = [&](int sb, const uint32_t (&w)[4][TW]) {
            uint32_t hw[4] = {0, 0, 0, 0};   // per row: the metadata nibbles of this thread's groups, at their place in the tile's 16 bits
#pragma unroll
            for (int j = 0; j < GPT; j++) {
                uint32_t out[4];
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const uint32_t *wg = &w[r][j * NW];
                    uint32_t h[4];
                    bool nz[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const uint32_t cc = cand[j][c];
                        // half cc of the group's NW words: a binary select tree down to a pair of words, then one byte permute
                        uint32_t lo, hi;
                        if (NW == 2) {
                            lo = wg[0]; hi = wg[1];
                        } else if (NW == 4) {
                            const bool up = (cc & 4u) != 0;
                            lo = up ? wg[2] : wg[0];
                            hi = up ? wg[3] : wg[1];
                        } else {
                            const bool up8 = (cc & 8u) != 0, up4 = (cc & 4u) != 0;
                            const uint32_t a0 = up8 ? wg[4] : wg[0], a1 = up8 ? wg[5] : wg[1];
                            const uint32_t a2 = up8 ? wg[6] : wg[2], a3 = up8 ? wg[7] : wg[3];
                            lo = up4 ? a2 : a0;
                            hi = up4 ? a3 : a1;
                        }
                        const uint32_t h2 = (cc & 3u) * 2u;
                        h[c] = __byte_perm(lo, hi, ((h2 + 1u) << 4) | h2);   // the half in the low 16 bits (the upper 16 are not used)
                        nz[c] = (h[c] & 0x7FFFu) != 0;                                // kept entries are the non-zero values
                    }
                    // exactly two candidates are non-zero in a valid matrix: the first from the front and the first from the back
                    const uint32_t v0 = nz[0] ? h[0] : (nz[1] ? h[1] : h[2]), i0 = nz[0] ? 0u : (nz[1] ? 1u : 2u);
                    const uint32_t v1 = nz[3] ? h[3] : (nz[2] ? h[2] : h[1]), i1 = nz[3] ? 3u : (nz[2] ? 2u : 1u);
                    const int cnt = (int)nz[0] + (int)nz[1] + (int)nz[2] + (int)nz[3];
                    const bool good = cnt == 2 && okmask[j] != 0;
                    bad += (valid && !good);
                    // fewer than two kept entries leave zeros in the open slots, more than two keep the first two (as the scalar form does)
                    uint32_t o, nib;
                    if (cnt == 2) {
                        o = __byte_perm(v0, v1, 0x5410u);   // low halves of both
                        nib = i0 | (i1 << 2);
                    } else {
                        o = 0; nib = 0;
                        int pos = 0;
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            if (nz[c]) {
                                if (pos < 2) { o |= (h[c] & 0xFFFFu) << (16 * pos); nib |= (uint32_t)c << (pos * 2); }
                                pos++;
                            }
                    }
                    out[r] = o & okmask[j];
                    hw[r] |= (nib & okmask[j]) << ((g0 + j) * 4);
                }
                // rows 4*sb .. 4*sb+3 of group g0 + j: one 16-byte piece of [sub-block][group][row][slot]
                if (valid) vdst[sb * 4 + j] = make_uint4(out[0], out[1], out[2], out[3]);
            }
            // the tile's 16 metadata bits per row, two rows per word: OR over the lanes of the tile
            uint32_t m01 = hw[0] | (hw[1] << 16), m23 = hw[2] | (hw[3] << 16);
#pragma unroll
            for (int o = 1; o < TL; o <<= 1) {
                m01 |= __shfl_xor_sync(0xffffffffu, m01, o);
                m23 |= __shfl_xor_sync(0xffffffffu, m23, o);
            }
            if (TL == 4) {
                if (tli == sb) { keep[0] = m01; keep[1] = m23; }
            } else {
                if (tli == (sb >> 1)) { keep[(sb & 1) * 2] = m01; keep[(sb & 1) * 2 + 1] = m23; }
            }
        };
        load4(row0, 1, wb);
        work(0, wa);
        load4(row0, 2, wa);
        work(1, wb);
        load4(row0, 3, wb);
        work(2, wa);
        load4(next_row0, 0, wa);   // the next item's first rows (the last item loads its own again: in bounds, unused)
        work(3, wb);
        row0 = next_row0;
        // the strip's half of the tile's 16 metadata words (rows 16*(strip & 1) ..): 32 bytes, one sector per tile
        uint32_t *mdst = meta + (int64_t)(strip >> 1) * 16 * tiles + (int64_t)T * 16 + (strip & 1u) * 8;
        if (valid) {
            if (TL == 4) *reinterpret_cast<uint2 *>(mdst + tli * 2) = make_uint2(keep[0], keep[1]);
            else *reinterpret_cast<uint4 *>(mdst + tli * 4) = make_uint4(keep[0], keep[1], keep[2], keep[3]);
        }
    }
    if (violations != nullptr) {
        for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
        if (lane == 0 && bad) atomicAdd(violations, (unsigned long long)bad);
    }
}

// one resident wave of the register-form compressor on the current device (cached per kernel and device)
template <int M_>
static int compress_direct_wave()
{
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int per_sm = 0, sms = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, compress_direct_kernel<M_>, 256, 0);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = (per_sm > 0 && sms > 0) ? per_sm * sms : 148 * 4;
    }
    return cached[dev];
}

cudaError_t launch_compress(const void *dense, int64_t ldd, const int32_t *mask, const uint32_t *colloc, int M, int K, int V, int m,
                            void *values, uint32_t *meta, unsigned long long *violations, cudaStream_t stream)
{
    const int64_t Ksp = ksp_of(K, m);
    const int threads = 256;
    // register form: no mask, whole tiles, 16-byte aligned rows and outputs
    if (!mask && (m == 4 || m == 8 || m == 16) && K % (4 * m) == 0 && Ksp == (int64_t)K / m * 2 && M % 16 == 0 && V % 16 == 0 && ldd % 8 == 0 &&
        ((uintptr_t)dense & 15) == 0 && ((uintptr_t)values & 15) == 0 && ((uintptr_t)colloc & 15) == 0 && ((uintptr_t)meta & 15) == 0) {
        const int tiles = (int)(Ksp / 8);
        const int tiles_per_item = m == 4 ? 8 * 16 : 8 * 8;   // 8 warps x tiles per warp
        const int64_t spans = (tiles + tiles_per_item - 1) / tiles_per_item, items = (int64_t)(M / 16) * spans;
        if (items < ((int64_t)1 << 31)) {
            const int wave = m == 4 ? compress_direct_wave<4>() : m == 8 ? compress_direct_wave<8>() : compress_direct_wave<16>();
            const unsigned blocks = items < wave ? (unsigned)items : (unsigned)wave;
            if (m == 4)
                compress_direct_kernel<4><<<blocks, threads, 0, stream>>>((const __half *)dense, ldd, colloc, V, tiles, (uint32_t)spans, (uint32_t)items, (uint32_t *)values, meta, violations);
            else if (m == 8)
                compress_direct_kernel<8><<<blocks, threads, 0, stream>>>((const __half *)dense, ldd, colloc, V, tiles, (uint32_t)spans, (uint32_t)items, (uint32_t *)values, meta, violations);
            else
                compress_direct_kernel<16><<<blocks, threads, 0, stream>>>((const __half *)dense, ldd, colloc, V, tiles, (uint32_t)spans, (uint32_t)items, (uint32_t *)values, meta, violations);
            return cudaGetLastError();
        }
    }
    const bool aligned = ldd % 4 == 0 && ((uintptr_t)dense & 7) == 0 && ((uintptr_t)mask & 7) == 0 && ((uintptr_t)meta & 15) == 0 &&
                         m <= 128 && M % 32 == 0 && V % 32 == 0;
    if (aligned) {
        const int TS = m >= 128 ? 1 : (m <= 8 ? 16 : 128 / m);  // at most 512 columns per chunk
        const int span = TS * 4 * m;
        const size_t smem = (size_t)(2 * TS * 64 + TS * 16) * 4 + (size_t)2 * 32 * (span + 4) * 2 + (mask ? (size_t)32 * (((span / 2 + 7) & ~7) + 4) : 0);
        const int64_t chunks = (int64_t)(M / 32) * ((Ksp / 8 + TS - 1) / TS);
        int64_t blocks = chunks < (int64_t)148 * 3 ? chunks : (int64_t)148 * 3;
        // up to ~83 KiB: two input buffers, the output staging and the mask bits
        cudaError_t e = mask ? cudaFuncSetAttribute(compress_tiled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)
                             : cudaFuncSetAttribute(compress_tiled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return e;
        if (blocks < 1) blocks = 1;
        if (mask)
            compress_tiled_kernel<true><<<(unsigned)blocks, threads, smem, stream>>>((const __half *)dense, ldd, mask, colloc, M, K, V, m, Ksp, TS,
                                                                                   (uint32_t *)values, meta, violations);
        else
            compress_tiled_kernel<false><<<(unsigned)blocks, threads, smem, stream>>>((const __half *)dense, ldd, mask, colloc, M, K, V, m, Ksp, TS,
                                                                                    (uint32_t *)values, meta, violations);
        return cudaGetLastError();
    }
    const int64_t total = (int64_t)(M / 2) * (Ksp / 8);
    int64_t blocks = (total + threads - 1) / threads;
    const int64_t cap = (int64_t)148 * 64;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (mask)
        compress_kernel<true><<<(unsigned)blocks, threads, 0, stream>>>((const __half *)dense, ldd, mask, colloc, M, K, V, m, Ksp,
                                                                       (__half *)values, meta, violations);
    else
        compress_kernel<false><<<(unsigned)blocks, threads, 0, stream>>>((const __half *)dense, ldd, mask, colloc, M, K, V, m, Ksp,
                                                                        (__half *)values, meta, violations);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Decompressor, general form (Format_sr_nm<T>::to_dense, format_sr_nm.cpp:327-417).  The output is zero-filled by
// the caller side of the launch; one thread scatters the two values of one (row, group), slot 0
// first, so a padded slot overwrites exactly as the reference's loop order does.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) decompress_kernel(const __half *__restrict__ values, const uint32_t *__restrict__ meta,
                                                         const uint32_t *__restrict__ colloc, int M, int K, int V, int m, int64_t Ksp,
                                                         __half *__restrict__ dense, int64_t ldd)
{
    const int64_t G = Ksp / 2;
    const int64_t total = (int64_t)M * G;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / G;
        const int64_t g = idx - r * G;
        const uint32_t w = meta[meta_index(r, g, Ksp)];
        const uint32_t *c4 = colloc + (r / V) * G * 4 + g * 4;
#pragma unroll
        for (int s = 0; s < 2; s++) {
            const uint32_t sel = (w >> meta_shift(r, g, s)) & 3u;
            const int64_t col = g * m + (int64_t)c4[sel];
            if (col < K) dense[r * ldd + col] = values[values_index(r, g, s, Ksp)];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Tiled decompressor (the one normally used): the mirror image of compress_tiled_kernel.  A CTA takes 32 rows x
// TS tiles: the values (TS * 256 contiguous bytes per 16 rows) and metadata (TS * 64 bytes) come in with 16-byte
// loads, lane = row / warp = tile scatters the two values of every (row, group) into a zeroed shared-memory image
// of the 32 dense row segments (slot 0 first, like the general kernel), and the image leaves with 8-byte stores.
// Every output element is written exactly once, so no memset pass is needed.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) decompress_tiled_kernel(const uint32_t *__restrict__ values, const uint32_t *__restrict__ meta,
                                                               const uint32_t *__restrict__ colloc, int M, int K, int V, int m, int64_t Ksp, int TS,
                                                               __half *__restrict__ dense, int64_t ldd)
{
    extern __shared__ __align__(16) uint8_t csm[];
    const int span = TS * 4 * m;
    const int pitch = span + 4;  // halves; rows 8-byte aligned, pitch / 2 = 2 mod 32
    uint32_t *val_s = reinterpret_cast<uint32_t *>(csm);                 // [2][TS][64]
    uint32_t *meta_s = val_s + 2 * TS * 64;                              // [TS][16]
    unsigned short *out_s = reinterpret_cast<unsigned short *>(meta_s + TS * 16);  // [32][pitch]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tiles = Ksp / 8;
    const int spans = (int)((tiles + TS - 1) / TS);
    const int64_t chunks = (int64_t)(M / 32) * spans;
    for (int64_t ch = blockIdx.x; ch < chunks; ch += gridDim.x) {
        const int64_t rc = ch / spans;
        const int sp = (int)(ch - rc * spans);
        const int64_t R0 = rc * 32;
        const int64_t t0 = (int64_t)sp * TS;
        const int tcount = (int)(tiles - t0 < TS ? tiles - t0 : TS);
        const int64_t c0 = t0 * 4 * m;
        const int valid = (int)(c0 >= K ? 0 : (K - c0 < span ? K - c0 : span));
        // ---- compressed arrays -> shared memory, dense image zeroed
        const int vq = tcount * 16;
        for (int i = threadIdx.x; i < 2 * vq; i += 256) {
            const int rg = i >= vq ? 1 : 0;
            const int k = i - rg * vq;
            reinterpret_cast<uint4 *>(val_s + rg * TS * 64)[k] = __ldg(reinterpret_cast<const uint4 *>(values + ((R0 / 16 + rg) * 16 * Ksp + t0 * 128) / 2) + k);
        }
        for (int i = threadIdx.x; i < tcount * 4; i += 256)
            reinterpret_cast<uint4 *>(meta_s)[i] = __ldg(reinterpret_cast<const uint4 *>(meta + (R0 / 32) * 16 * tiles + t0 * 16) + i);
        for (int i = threadIdx.x; i < 32 * pitch / 4; i += 256) reinterpret_cast<uint2 *>(out_s)[i] = make_uint2(0u, 0u);
        __syncthreads();
        // ---- lane = row, warp = tile
        const uint32_t *crow = colloc + (R0 / V) * (Ksp / 2) * 4;
        unsigned short *my_out = out_s + lane * pitch;
        for (int tl = warp; tl < tcount; tl += 8) {
            const uint32_t hw = (meta_s[tl * 16 + (lane >> 1)] >> ((lane & 1) * 16)) & 0xFFFFu;
            const uint32_t *vsrc = val_s + ((lane >> 4) * TS + tl) * 64 + ((lane & 15) >> 2) * 16 + (lane & 3);
            const uint4 *c4p = reinterpret_cast<const uint4 *>(crow + (t0 + tl) * 16);
#pragma unroll
            for (int gi = 0; gi < 4; gi++) {
                const uint4 c4 = __ldg(c4p + gi);
                const int cand[4] = {(int)c4.x, (int)c4.y, (int)c4.z, (int)c4.w};
                const int lg = (tl * 4 + gi) * m;
                const uint32_t two = vsrc[gi * 4];
#pragma unroll
                for (int sl = 0; sl < 2; sl++) {
                    const int sel = (int)((hw >> (gi * 4 + sl * 2)) & 3u);
                    const int lc = lg + (sel == 0 ? cand[0] : sel == 1 ? cand[1] : sel == 2 ? cand[2] : cand[3]);
                    if (lc < valid) my_out[lc] = (unsigned short)(two >> (16 * sl));
                }
            }
        }
        __syncthreads();
        // ---- dense image -> global memory
        const int nq = valid / 4;  // whole 8-byte pieces per row
        for (int r = warp; r < 32; r += 8) {
            __half *drow = dense + (R0 + r) * ldd + c0;
            const unsigned short *srow = out_s + r * pitch;
            for (int q = lane; q < nq; q += 32) reinterpret_cast<uint2 *>(drow)[q] = reinterpret_cast<const uint2 *>(srow)[q];
            for (int c = nq * 4 + lane; c < valid; c += 32) drow[c] = __ushort_as_half(srow[c]);
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------
// Decompressor, register form: the mirror image of compress_direct_kernel (used for m in {4, 8}, whole
// tiles, V % 16 == 0, aligned rows).  Lanes lie along the row; a thread owns one group (two for m = 4) of the 16 rows of
// a strip.  For four consecutive rows its kept pairs are one 16-byte piece of the value array and its metadata nibbles
// sit in the tile's two metadata words of those rows; it rebuilds the m halves of the group in registers (zeros, slot 0,
// then slot 1, so a padded slot overwrites as in the reference's loop order) and stores them with 16-byte stores: a
// warp writes 512 contiguous bytes of a row (1 KiB for m = 16).  Every output element is written exactly once.
// ------------------------------------------------------------------------------------------------
template <int M_>
__global__ void __launch_bounds__(256) decompress_direct_kernel(const uint32_t *__restrict__ values, const uint32_t *__restrict__ meta,
                                                                const uint32_t *__restrict__ colloc, int V, int tiles, uint32_t spans,
                                                                uint32_t items, __half *__restrict__ dense, int64_t ldd)
{
    constexpr int NW = M_ / 2;             // 32-bit words per group
    constexpr int GPT = M_ == 4 ? 2 : 1;   // groups per thread
    constexpr int TW = GPT * NW;           // words per thread and row
    constexpr int TL = 4 / GPT;            // lanes per tile
    constexpr int TPW = 32 / TL;           // tiles per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g0 = (lane % TL) * GPT;
    const int64_t Ksp = (int64_t)tiles * 8;
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t strip = item / spans;
        const int T = (int)(item - strip * spans) * (8 * TPW) + warp * TPW + lane / TL;
        if (T >= tiles) continue;   // no exchange between lanes: threads past the last tile have nothing to do
        const int64_t G = (int64_t)T * 4 + g0;
        // the candidates of a group as four bytes of one word: candidate `sel` is one byte permute away
        uint32_t candpack[GPT];
        {
            const uint4 *c4p = reinterpret_cast<const uint4 *>(colloc + ((int64_t)(strip * 16u / (uint32_t)V) * (Ksp / 2) + G) * 4);
#pragma unroll
            for (int j = 0; j < GPT; j++) {
                const uint4 c4 = __ldg(c4p + j);
                candpack[j] = (c4.x & 0xFFu) | ((c4.y & 0xFFu) << 8) | ((c4.z & 0xFFu) << 16) | ((c4.w & 0xFFu) << 24);
            }
        }
        const uint4 *vsrc = reinterpret_cast<const uint4 *>(values) + ((int64_t)strip * 16 * Ksp + (int64_t)T * 128) / 8 + g0;
        const uint4 *msrc = reinterpret_cast<const uint4 *>(meta + (int64_t)(strip >> 1) * 16 * tiles + (int64_t)T * 16 + (strip & 1u) * 8);
        uint4 vals[4][GPT];
#pragma unroll
        for (int sb = 0; sb < 4; sb++)
#pragma unroll
            for (int j = 0; j < GPT; j++) vals[sb][j] = __ldg(vsrc + sb * 4 + j);
        const uint4 ma = __ldg(msrc), mb = __ldg(msrc + 1);
        const uint32_t mw[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};   // word 2*sb + (r >> 1): rows r, r+1 of sub-block sb
        __half *drow0 = dense + (int64_t)strip * 16 * ldd + G * M_;
#pragma unroll
        for (int sb = 0; sb < 4; sb++) {
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const uint32_t hw = mw[sb * 2 + (r >> 1)] >> ((r & 1) * 16);
                uint32_t w[TW];
#pragma unroll
                for (int j = 0; j < GPT; j++) {
                    const uint32_t two = r == 0 ? vals[sb][j].x : r == 1 ? vals[sb][j].y : r == 2 ? vals[sb][j].z : vals[sb][j].w;
                    const uint32_t nib = hw >> ((g0 + j) * 4);
                    const uint32_t p0 = __byte_perm(candpack[j], 0u, 0x4440u | (nib & 3u));          // column of slot 0 inside the group
                    const uint32_t p1 = __byte_perm(candpack[j], 0u, 0x4440u | ((nib >> 2) & 3u));   // column of slot 1
                    const uint32_t lo0 = two & 0xFFFFu, hi0 = two << 16;          // slot 0 as a low / high half
                    const uint32_t lo1 = two >> 16, hi1 = two & 0xFFFF0000u;      // slot 1
#pragma unroll
                    for (int k = 0; k < NW; k++) {
                        uint32_t x = 0;
                        if ((p0 >> 1) == (uint32_t)k) x = (p0 & 1u) ? hi0 : lo0;
                        if ((p1 >> 1) == (uint32_t)k) x = (p1 & 1u) ? ((x & 0xFFFFu) | hi1) : ((x & 0xFFFF0000u) | lo1);
                        w[j * NW + k] = x;
                    }
                }
                uint4 *dst = reinterpret_cast<uint4 *>(drow0 + (int64_t)(sb * 4 + r) * ldd);
#pragma unroll
                for (int i = 0; i < TW / 4; i++) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            }
        }
    }
}

template <int M_>
static int decompress_direct_wave()
{
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int per_sm = 0, sms = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decompress_direct_kernel<M_>, 256, 0);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = (per_sm > 0 && sms > 0) ? per_sm * sms : 148 * 4;
    }
    return cached[dev];
}

cudaError_t launch_decompress(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int m,
                              void *dense, int64_t ldd, cudaStream_t stream)
{
    const int64_t Ksp = ksp_of(K, m);
    // register form: whole tiles, 16-byte aligned rows and arrays (m = 16 measured slower than the tiled kernel: a lane's
    // 32 bytes per row leave through two strided 16-byte stores)
    if ((m == 4 || m == 8) && K % (4 * m) == 0 && Ksp == (int64_t)K / m * 2 && M % 16 == 0 && V % 16 == 0 && ldd % 8 == 0 &&
        ((uintptr_t)dense & 15) == 0 && ((uintptr_t)values & 15) == 0 && ((uintptr_t)colloc & 15) == 0 && ((uintptr_t)meta & 15) == 0) {
        const int tiles = (int)(Ksp / 8);
        const int tiles_per_item = m == 4 ? 8 * 16 : 8 * 8;   // 8 warps x tiles per warp
        const int64_t spans = (tiles + tiles_per_item - 1) / tiles_per_item, items = (int64_t)(M / 16) * spans;
        if (items < ((int64_t)1 << 31)) {
            const int wave = m == 4 ? decompress_direct_wave<4>() : decompress_direct_wave<8>();
            const unsigned blocks = items < wave ? (unsigned)items : (unsigned)wave;
            if (m == 4)
                decompress_direct_kernel<4><<<blocks, 256, 0, stream>>>((const uint32_t *)values, meta, colloc, V, tiles, (uint32_t)spans, (uint32_t)items, (__half *)dense, ldd);
            else
                decompress_direct_kernel<8><<<blocks, 256, 0, stream>>>((const uint32_t *)values, meta, colloc, V, tiles, (uint32_t)spans, (uint32_t)items, (__half *)dense, ldd);
            return cudaGetLastError();
        }
    }
    const bool aligned = ldd % 4 == 0 && ((uintptr_t)dense & 7) == 0 && ((uintptr_t)values & 15) == 0 && ((uintptr_t)meta & 15) == 0 &&
                         m <= 128 && M % 32 == 0 && V % 32 == 0;
    if (aligned) {
        const int TS = m >= 128 ? 1 : (m <= 8 ? 16 : 128 / m);
        const int span = TS * 4 * m;
        const size_t smem = (size_t)(2 * TS * 64 + TS * 16) * 4 + (size_t)32 * (span + 4) * 2;
        const int64_t chunks = (int64_t)(M / 32) * ((Ksp / 8 + TS - 1) / TS);
        int64_t blocks = chunks < (int64_t)148 * 5 ? chunks : (int64_t)148 * 5;
        if (blocks < 1) blocks = 1;
        cudaError_t e = cudaFuncSetAttribute(decompress_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return e;
        decompress_tiled_kernel<<<(unsigned)blocks, 256, smem, stream>>>((const uint32_t *)values, meta, colloc, M, K, V, m, Ksp, TS,
                                                                         (__half *)dense, ldd);
        return cudaGetLastError();
    }
    cudaError_t e = cudaMemset2DAsync(dense, (size_t)ldd * 2, 0, (size_t)K * 2, (size_t)M, stream);
    if (e != cudaSuccess) return e;
    const int64_t total = (int64_t)M * (Ksp / 2);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)148 * 64;
    if (blocks > cap) blocks = cap;
    decompress_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __half *)values, meta, colloc, M, K, V, m, Ksp, (__half *)dense, ldd);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Re-pack into the kernel-private layout (see vnm_common.cuh).  One thread writes one 16-byte chunk:
// chunks [0, 1024) of a block are the swizzled value image, chunks [1024, 1152) the metadata image.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prepare_am_kernel(const __half *__restrict__ values, const uint32_t *__restrict__ meta, int M,
                                                         int64_t Ksp, int mtiles, int ktiles, uint4 *__restrict__ am)
{
    const int chunks_per_block = AM_BLOCK_BYTES / 16;  // 1152
    const int64_t total = (int64_t)mtiles * ktiles * chunks_per_block;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t blk = idx / chunks_per_block;
        const int ch = (int)(idx - blk * chunks_per_block);
        const int mt = (int)(blk / ktiles);
        const int kt = (int)(blk - (int64_t)mt * ktiles);
        uint4 o = make_uint4(0, 0, 0, 0);
        if (ch < A_IMG_BYTES / 16) {
            const int i = ch >> 3;                  // MMA row inside the tile
            const int cphys = ch & 7;               // stored chunk
            const int c = cphys ^ (i & 7);          // logical chunk = 8 compressed columns = one reference tile
            const int64_t r = (int64_t)mt * TILE_M + mma_row_to_actual(i);
            const int64_t t = (int64_t)kt * 8 + c;  // reference tile index (four groups)
            if (r < M && t < Ksp / 8) {
                const __half *src = values + (r / 16) * 16 * Ksp + t * 128 + ((r % 16) / 4) * 32 + (r % 4) * 2;
                uint32_t w[4];
#pragma unroll
                for (int gi = 0; gi < 4; gi++) w[gi] = *reinterpret_cast<const uint32_t *>(src + gi * 8);
                o = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
            const int lane = ch - A_IMG_BYTES / 16;  // tensor-memory lane 0..127
            const int m0 = lane & 7, k1 = (lane >> 3) & 1, m2 = lane >> 4;
            const int64_t r = (int64_t)mt * TILE_M + m2 * 16 + m0 * 2;  // even row of the pair
            uint32_t w[4];
#pragma unroll
            for (int kb = 0; kb < 4; kb++) {
                const int64_t t = (int64_t)kt * 8 + kb * 2 + k1;
                // padding: positions (0,1) in every group, a valid 2:4 pattern for zero values
                w[kb] = (r < M && t < Ksp / 8) ? meta[(r / 32) * 16 * (Ksp / 8) + t * 16 + (r % 32) / 2] : 0x44444444u;
            }
            o = make_uint4(w[0], w[1], w[2], w[3]);
        }
        am[idx] = o;
    }
}

// Absolute B rows per (V-block, group); groups are padded to whole k-tiles and V-blocks to whole row tiles.
__global__ void __launch_bounds__(256) prepare_rows_kernel(const uint32_t *__restrict__ colloc, int M, int K, int V, int m, int64_t Ksp,
                                                           int vblocks_padded, int ktiles, int4 *__restrict__ rows)
{
    const int64_t gpad = (int64_t)ktiles * KT_GROUPS;
    const int64_t total = (int64_t)vblocks_padded * gpad;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t vb = idx / gpad;
        const int64_t g = idx - vb * gpad;
        int4 o = make_int4(K, K, K, K);
        if (vb < M / V && g < Ksp / 2) {
            const uint4 c4 = *reinterpret_cast<const uint4 *>(colloc + vb * (Ksp / 2) * 4 + g * 4);
            const int64_t base = g * m;
            const int64_t a = base + c4.x, b = base + c4.y, c = base + c4.z, d = base + c4.w;
            o.x = a < K ? (int)a : K;
            o.y = b < K ? (int)b : K;
            o.z = c < K ? (int)c : K;
            o.w = d < K ? (int)d : K;
        }
        rows[idx] = o;
    }
}

// ------------------------------------------------------------------------------------------------
// "Dense-B" re-pack: the V:2:m pattern re-expressed as plain 2:4 over ALL K columns.
// A row keeps two entries per group of m columns, so any aligned chunk of four original columns
// (m % 4 == 0: chunks never straddle groups) holds at most two of them -- a valid 2:4 pattern once the
// missing slots are filled with explicit zeros.  The product can then read B as ordinary 64-row tiles
// that every vector block shares (no per-block gather, no lane masks), at the price of m/4 times the MMA
// work.  Same block format as prepare_am_kernel, but a k-tile now covers 128 ORIGINAL columns.
// One thread handles one (row pair, 16 original columns): two 16-byte value chunks and one metadata word.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prepare_dense_b_kernel(const __half *__restrict__ values, const uint32_t *__restrict__ meta,
                                                              const uint32_t *__restrict__ colloc, int M, int K, int V, int m, int64_t Ksp,
                                                              int mtiles, int ktiles, uint8_t *__restrict__ am)
{
    const int64_t total = (int64_t)mtiles * ktiles * 64 * 8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int q = (int)(idx & 7);          // 16-column slab of the 128-column k-tile
        const int pr = (int)((idx >> 3) & 63);  // row pair inside the 128-row tile
        const int64_t blk = idx >> 9;
        const int mt = (int)(blk / ktiles);
        const int kt = (int)(blk - (int64_t)mt * ktiles);
        uint8_t *block = am + blk * AM_BLOCK_BYTES;
        uint32_t word = 0;
        const int i0 = actual_to_mma_row(2 * pr);  // MMA row of the even row; the odd row sits 8 rows further
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t r = (int64_t)mt * TILE_M + 2 * pr + h;
            unsigned short v8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            uint32_t nib16 = 0;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int64_t cb = (int64_t)kt * 128 + q * 16 + c * 4;  // first original column of the chunk
                int npos = 0;
                uint32_t pos[2] = {0, 1};
                unsigned short val[2] = {0, 0};
                if (r < M && cb < K) {
                    const int64_t g = cb / m;
                    const int o0 = (int)(cb - g * m);
                    const uint32_t w = meta[meta_index(r, g, Ksp)];
                    const uint32_t *c4 = colloc + (r / V) * (Ksp / 2) * 4 + g * 4;
#pragma unroll
                    for (int sl = 0; sl < 2; sl++) {
                        const uint32_t sel = (w >> meta_shift(r, g, sl)) & 3u;
                        const int off = (int)c4[sel] - o0;
                        if (off >= 0 && off < 4 && npos < 2 && cb + off < K) {
                            pos[npos] = (uint32_t)off;
                            val[npos] = __half_as_ushort(values[values_index(r, g, sl, Ksp)]);
                            npos++;
                        }
                    }
                }
                if (npos == 1) {  // partner slot with an explicit zero, positions kept ascending
                    if (pos[0] == 3) { pos[1] = 3; pos[0] = 2; val[1] = val[0]; val[0] = 0; }
                    else { pos[1] = pos[0] + 1; val[1] = 0; }
                } else if (npos == 0) {
                    pos[0] = 0; pos[1] = 1;
                } else if (pos[0] == pos[1]) {  // duplicate offsets only arise from padded slots (zero values)
                    if (pos[0] == 3) pos[0] = 2; else pos[1] = pos[0] + 1;
                }
                v8[2 * c] = val[0];
                v8[2 * c + 1] = val[1];
                nib16 |= (pos[0] | (pos[1] << 2)) << (4 * c);
            }
            word |= nib16 << (16 * h);
            const int i = i0 + 8 * h;
            uint4 o;
            o.x = (uint32_t)v8[0] | ((uint32_t)v8[1] << 16);
            o.y = (uint32_t)v8[2] | ((uint32_t)v8[3] << 16);
            o.z = (uint32_t)v8[4] | ((uint32_t)v8[5] << 16);
            o.w = (uint32_t)v8[6] | ((uint32_t)v8[7] << 16);
            *reinterpret_cast<uint4 *>(block + i * 128 + ((q ^ (i & 7)) << 4)) = o;
        }
        const int lane = (i0 & 7) + 8 * (q & 1) + 16 * (i0 >> 4);
        *reinterpret_cast<uint32_t *>(block + A_IMG_BYTES + (lane * 4 + (q >> 1)) * 4) = word;
    }
}

// Row table of the dense-B form: stage j of a tile starts at original row 64*j.
__global__ void __launch_bounds__(256) prepare_dense_b_rows_kernel(int K, int mtiles, int ktiles, int4 *__restrict__ rows)
{
    const int64_t per_tile = (int64_t)ktiles * KT_GROUPS;
    const int64_t total = (int64_t)mtiles * per_tile;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t g = idx % per_tile;
        const int64_t k = g * 4;
        rows[idx] = k < K ? make_int4((int)k, (int)k + 1, (int)k + 2, (int)k + 3) : make_int4(K, K, K, K);
    }
}

cudaError_t launch_prepare_dense_b(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int m,
                                   void *am, void *rows, int mtiles, int ktiles, cudaStream_t stream)
{
    const int64_t Ksp = ksp_of(K, m);
    const int64_t cap = (int64_t)148 * 64;
    {
        const int64_t total = (int64_t)mtiles * ktiles * 512;
        int64_t blocks = (total + 255) / 256;
        if (blocks > cap) blocks = cap;
        prepare_dense_b_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __half *)values, meta, colloc, M, K, V, m, Ksp, mtiles, ktiles,
                                                                   (uint8_t *)am);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    {
        const int64_t total = (int64_t)mtiles * ktiles * KT_GROUPS;
        int64_t blocks = (total + 255) / 256;
        if (blocks > cap) blocks = cap;
        prepare_dense_b_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(K, mtiles, ktiles, (int4 *)rows);
        return cudaGetLastError();
    }
}

cudaError_t launch_prepare(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int m,
                           void *am, void *rows, int mtiles, int ktiles, int vblocks_padded, cudaStream_t stream)
{
    const int64_t Ksp = ksp_of(K, m);
    {
        const int64_t total = (int64_t)mtiles * ktiles * (AM_BLOCK_BYTES / 16);
        int64_t blocks = (total + 255) / 256;
        const int64_t cap = (int64_t)148 * 64;
        if (blocks > cap) blocks = cap;
        prepare_am_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __half *)values, meta, M, Ksp, mtiles, ktiles, (uint4 *)am);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    {
        const int64_t total = (int64_t)vblocks_padded * ktiles * KT_GROUPS;
        int64_t blocks = (total + 255) / 256;
        const int64_t cap = (int64_t)148 * 64;
        if (blocks > cap) blocks = cap;
        prepare_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(colloc, M, K, V, m, Ksp, vblocks_padded, ktiles, (int4 *)rows);
        return cudaGetLastError();
    }
}

}  // namespace vnm
