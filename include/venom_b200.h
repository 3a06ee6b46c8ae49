/*
 * venom_b200 C ABI: V:N:M (VENOM) sparse x dense matrix product for NVIDIA B200 (sm_100a).
 *
 * Every entry point returns 0 on success and a non-zero VNM_ERR_* code otherwise; none of them exits
 * or throws.  vnm_last_error_string() returns the message of the last failure on the calling thread.
 * All data pointers are DEVICE pointers owned by the caller unless a name ends in _host.  `stream`
 * is a cudaStream_t passed as void* (NULL = the legacy default stream); work is asynchronous on it.
 *
 * Storage format ("reference format"): the three arrays of the reference's Format_sr_nm<half>
 * (src/format/format_sr_nm.cpp:53-60 of UDC-GAC/venom), bit-for-bit:
 *   values   fp16[M * Ksp]              Ksp = ROUND_UP(ceil(K/m) * 2, 16)
 *   metadata u32 [(M/2) * (Ksp/8)]      2-bit positions, 16 per word, two rows per word
 *   colloc   u32 [(M/V) * (Ksp/2) * 4]  four ascending column offsets in [0,m) per V x m block
 * n must be 2, m >= 4, V % 32 == 0, M % V == 0.  The SpMM additionally needs V in {32, 64, 128}.
 */
#ifndef VENOM_B200_H_
#define VENOM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    VNM_OK = 0,
    VNM_ERR_BAD_ARG = 1,     /* shape / alignment / null pointer */
    VNM_ERR_CUDA = 2,        /* a CUDA runtime or driver call failed */
    VNM_ERR_UNSUPPORTED = 3, /* valid format, but not implemented by the kernels (e.g. V = 96) */
    VNM_ERR_DEVICE_TIMEOUT = 4 /* a bounded device-side wait gave up; the context stays usable */
};

/* Output layouts of vnm_spmm_f16. */
enum {
    VNM_LAYOUT_MN = 0, /* out[r * ldo + c]: [M, N] row-major, the CLI kernel's layout */
    VNM_LAYOUT_NM = 1  /* out[c * ldo + r] = fp16(acc) + bias[r]: [N, M] row-major, the torch op's layout */
};

typedef struct vnm_prepared_s *vnm_handle_t;

const char *vnm_last_error_string(void);
int vnm_version(void);

/* Array sizes of the reference format.
 * Replaces: the size arithmetic of Format_sr_nm<T>::init, src/format/format_sr_nm.cpp:53-60. */
int vnm_sizes(int M, int K, int V, int n, int m,
              int64_t *ksp, int64_t *values_elems, int64_t *meta_words, int64_t *colloc_words);

/* Dense -> V:N:M compressor and metadata packer (CUDA).
 * Replaces: Format_sr_nm<T>::init_from_dense -> to_sparse_sr_nm, src/format/format_sr_nm.cpp:108-149,
 * 419-543, and its Python twin to_sparse_sr_nm, end2end/grouped_nmv_tensor.py:487-675.
 *   dense   fp16 [M, K] row-major with leading dimension ldd (already pruned to the pattern)
 *   mask    optional int32 [M, K] (same ldd): kept entries are mask != 0 (Python twin); NULL = kept
 *           entries are the non-zero values (C++ reference)
 *   colloc  column-loc, an input exactly as in the reference
 *   values, meta  outputs, fully overwritten
 *   violations    optional device counter (unsigned 64-bit), incremented by the number of (row, group)
 *                 pairs that did not yield exactly two kept entries (the reference is undefined there;
 *                 this library keeps the first two and zero-fills missing slots) */
int vnm_compress_f16(const void *dense, int64_t ldd, const int32_t *mask, const uint32_t *colloc,
                     int M, int K, int V, int n, int m,
                     void *values, uint32_t *meta, unsigned long long *violations, void *stream);

/* Magnitude pruner (CUDA): picks, per V x m block, the four columns and, per row, the two entries that
 * maximise the kept |w| exactly as the reference's exhaustive search does.
 * Replaces: group_n_m2 / nm_vector_mask_sparsify, end2end/grouped_nmv_tensor.py:81-343,746-779.
 *   w       fp32 [M, K] weights (magnitudes are taken inside), leading dimension ldw
 *   mask    out, int32 [M, K] (leading dimension ldm): 1 = kept
 *   colloc  out, column-loc array of the format (padding groups are zeroed)
 * Needs K % m == 0 and V * m * 4 <= 48 KiB.  Bit-identical to the reference except when the second and third
 * largest |w| of a row of the winning column quadruple are exactly equal (the reference's pick then depends on
 * scratch state carried over from earlier blocks); the chosen columns never differ. */
int vnm_prune_magnitude_f32(const float *w, int64_t ldw, int M, int K, int V, int n, int m,
                            int32_t *mask, int64_t ldm, uint32_t *colloc, void *stream);

/* V:N:M -> dense decompressor (CUDA).  dense [M, K] fp16, leading dimension ldd, fully overwritten.
 * Replaces: Format_sr_nm<T>::to_dense, src/format/format_sr_nm.cpp:327-417. */
int vnm_decompress_f16(const void *values, const uint32_t *meta, const uint32_t *colloc,
                       int M, int K, int V, int n, int m, void *dense, int64_t ldd, void *stream);

/* Re-pack reference-format arrays into the kernel-private layout and return a handle that owns only
 * that private copy (the inputs may be freed once `stream` has drained).
 * Replaces: BlockwiseSpMatrix<half>::init_sparse + transform_and_sync_device,
 * include/spatha/block_sparse/spmm/blockwise_format.h:248-283,327-373, and
 * Format_sr_nm<T>::transform_and_sync_device, src/format/format_sr_nm.cpp:239-285. */
int vnm_prepare(const void *values, const uint32_t *meta, const uint32_t *colloc,
                int M, int K, int V, int n, int m, vnm_handle_t *handle, void *stream);
int vnm_prepared_bytes(int M, int K, int V, int n, int m, int64_t *bytes);
int vnm_destroy(vnm_handle_t handle);

/* Threading: a handle caches the tensor maps of the last dense operand and owns the host-buffer staging, so two
 * host threads must not call into the SAME handle at the same time (different handles are independent).  A handle
 * belongs to the device that was current in vnm_prepare; calls with another device current return VNM_ERR_BAD_ARG. */

/* out = A_vnm * B (+ bias), fp16 in, fp32 accumulate, fp16 out.
 * Replaces: SpmmNMInitFn_t / SpmmNMExecFn_t -> SpmmBlockwiseOp::initialize / operator(),
 * include/spatha/block_sparse/spmm/blockwise_op.h:90-161,209-246 (layout MN, bias must be NULL) and
 * spmm_cuda, end2end/spatha_mod/block_sparse/spmm/blockwise_library.cu:294-386 (layout NM + bias).
 *   B    fp16 [K, N] row-major, leading dimension ldb (ldb % 8 == 0, 16-byte aligned base)
 *   bias fp16 [M] or NULL (layout NM only)
 *   out  fp16, leading dimension ldo, 16-byte aligned base; ldo % 8 == 0 for layout MN, and for layout NM too when
 *        the operand is held in dense-B form (its epilogue writes with TMA stores)
 * N must be a multiple of 8. */
int vnm_spmm_f16(vnm_handle_t handle, const void *B, int64_t ldb, int N,
                 const void *bias, void *out, int64_t ldo, int layout, void *stream);

/* The same product stored to n_outs buffers of one geometry (1 <= n_outs <= VNM_MAX_OUTS; same ldo, layout and
 * alignment rules as `out` above): every output tile leaves shared memory through one TMA store per destination, so
 * the operands are read and multiplied once.  The destinations may be peer-mapped buffers of other GPUs -- this is the
 * store side of vnm_mgpu_spmm_gathered_p2p.  Operands held in dense-B form: both layouts; in gather form: layout NM with
 * ldo % 8 == 0 and 16-byte aligned buffers (the epilogue that leaves through TMA stores); VNM_ERR_UNSUPPORTED otherwise. */
#define VNM_MAX_OUTS 8
int vnm_spmm_f16_multi(vnm_handle_t handle, const void *B, int64_t ldb, int N, const void *bias,
                       void *const *outs, int n_outs, int64_t ldo, int layout, void *stream);

/* Same product with the dense operand given as Bt = B^T, i.e. [N, K] row-major with leading dimension ldbt
 * (the activation in its natural [tokens, features] layout), so the caller does not have to materialise the
 * transpose the reference's scripts make before every call (end2end/bert_pytorch.py:85-87,133).
 * Only for operands prepared in dense-B form (vnm_operand_form reports it); otherwise VNM_ERR_UNSUPPORTED. */
int vnm_spmm_f16_nk(vnm_handle_t handle, const void *Bt, int64_t ldbt, int N,
                    const void *bias, void *out, int64_t ldo, int layout, void *stream);
int vnm_operand_form(vnm_handle_t handle, int *dense_b);

/* Same product with HOST buffers: B (and bias) go up, the product runs on `stream`, the result comes back, and
 * the call returns after synchronising.  The columns are cut into up to eight slices so that the upload of one
 * slice, the product of the previous and the download of the one before run at the same time (two copy streams
 * per device, shared by all handles).  Device staging buffers are owned by the handle and grown on demand.
 * B_host [K, N] and out_host are dense row-major ([M,N] or [N,M]); pinned memory gives the overlap. */
int vnm_spmm_f16_host(vnm_handle_t handle, const void *B_host, int N, const void *bias_host,
                      void *out_host, int layout, void *stream);

/* The same call without the final wait: it returns once the copies and launches are queued, so that the
 * host-to-device copies of one product overlap the device-to-host copies of the one before (different
 * handles, or the same handle after vnm_host_wait).  out_host is valid after vnm_host_wait(handle); host buffers
 * should be pinned, otherwise the copies are synchronous anyway.  One outstanding call per handle.
 * No counterpart in the reference (its harness copies and computes in separate, blocking steps,
 * src/spmm/spatha_spmm.cpp:24-38,84-90). */
int vnm_spmm_f16_host_async(vnm_handle_t handle, const void *B_host, int N, const void *bias_host,
                            void *out_host, int layout, void *stream);
int vnm_host_wait(vnm_handle_t handle);

/* The same product for callers that cannot allocate device memory (no counterpart in the reference, whose
 * device format always comes from cudaMalloc).  Think of a serving process whose framework already owns
 * the whole device, a plug-in living inside another component's memory budget, or a loop that cannot take
 * the device-wide synchronisation of cudaMalloc / cudaFree.  The re-packed copy of the sparse operand,
 * which vnm_prepare would allocate, is written into an array built into the library instead
 * (VNM_NOALLOC_SCRATCH_BYTES per GPU that loads the library, held until the process exits), then the
 * product runs from it.  The call performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *   - takes the reference-format arrays directly (same meaning as in vnm_prepare) plus the arguments of
 *     vnm_spmm_f16; re-packs on every call, so it suits small operands and occasional calls;
 *   - operands whose re-packed form (about 1.13 x 2*M*Ksp bytes) exceeds the limit are rejected with
 *     VNM_ERR_UNSUPPORTED and a message naming both sizes;
 *   - the first call on a device also looks up the array's device address and sets kernel attributes: make
 *     that first call before starting any stream capture;
 *   - all calls on a device share the one array and it keeps the previous call's contents (the call clears
 *     what has to start at zero itself): two calls whose GPU work overlaps -- different streams or host
 *     threads -- race on it, so serialise them;
 *   - returns after the product has finished on `stream` (it synchronises the stream to read the device
 *     status word back); failures set vnm_last_error_string() like every entry point and also print one
 *     line to stderr. */
#define VNM_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
int vnm_spmm_f16_noalloc(const void *values, const uint32_t *meta, const uint32_t *colloc,
                         int M, int K, int V, int n, int m,
                         const void *B, int64_t ldb, int N, const void *bias, void *out, int64_t ldo, int layout, void *stream);

/* Reads and clears the sticky device-side status word of the handle (0 = no bounded wait ever gave
 * up).  Synchronises `stream`. */
int vnm_device_status(vnm_handle_t handle, int *status, void *stream);

/* Self-test of the failure path, without a fault: launches a two-warp kernel that waits, through the same bounded
 * wait as the product kernels (about two seconds), on a barrier that nothing signals.  The wait runs out, the
 * kernel records a status bit in this handle's status word and returns normally; the next vnm_device_status
 * reports VNM_ERR_DEVICE_TIMEOUT and clears the word, and the handle stays usable.  No counterpart in the
 * reference (its kernels have no waits that can fail). */
int vnm_selftest_wait_expiry(vnm_handle_t handle, void *stream);

/* Ablation switches.
 * Gather mode: how the selected rows of B reach shared memory.  0 = TMA tile::gather4, one group of four rows per
 * instruction (default for m > 4); 3 = 16-byte asynchronous copies (cp.async) issued per thread from the row table and
 * written straight into the swizzled operand layout (the staging the reference uses,
 * include/spatha/block_sparse/spmm/blockwise_kernel.h:868-881; measured slower than the TMA gather on B200, alone and
 * in any split with it, see vnm_set_gather_split); 1 = plain TMA tiles
 * of 64 consecutive rows, which is exact
 * for m == 4 (every row is selected; the default there) and otherwise removes the column-loc
 * indirection exactly like the reference's compile-time IDEAL_KERNEL experiment
 * (include/spatha/block_sparse/spmm/blockwise_kernel.h:328-642, row = nz_block_idx % 4 at :536);
 * 2 = B is not loaded at all (timing floor; results are meaningless).
 * Producer warps: 4 or 8 warps issue the gather loads (default 8). */
int vnm_set_gather_mode(vnm_handle_t handle, int mode);
/* Gather mode 3 only: of the 64 gathered rows of every stage, `tma_rows` (0, 16, 32 or 48) are fetched by TMA
 * tile::gather4 and the others by the per-thread copies, so that both paths into the SM are busy at once. */
int vnm_set_gather_split(vnm_handle_t handle, int tma_rows);
/* Epilogue of the V:N:M (gather) form.  0 (default): layout MN staged in shared memory and stored as full 128-bit
 * sectors; layout NM as fp16 stores from registers (several destinations -- vnm_spmm_f16_multi -- staged as [n][m] and
 * stored with TMA, boxes of 128 m x 32 n).  1 = layout MN: every thread stores its own row in 32-bit words, the
 * reference's OUT_32B experiment (include/spatha/block_sparse/common/epilogue.h:34-61, blockwise_kernel.h:911-943).
 * 2 = layout NM through TMA stores also for a single destination, where ldo % 8 == 0 and out is 16-byte aligned
 * (ablation: measured 1-4 % slower).  All give identical bits.  VNM_ERR_UNSUPPORTED for operands held in dense-B form,
 * whose epilogue always leaves through TMA stores. */
int vnm_set_epilogue(vnm_handle_t handle, int mode);

/* How vnm_prepare lays the sparse operand out for the kernel (process-wide, applies to later calls):
 *   AUTO     pick per (V, m) from measurements on B200 (default);
 *   GATHER   the V:N:M form: only the four selected rows of B per group are gathered per vector block;
 *   DENSE_B  the pattern re-expressed as plain 2:4 over all K columns (needs m % 4 == 0 and K % m == 0):
 *            B is read as ordinary tiles shared by all vector blocks, at m/4 times the MMA work.
 * Both forms give the same result up to fp32 summation order. */
enum { VNM_STRATEGY_AUTO = 0, VNM_STRATEGY_GATHER = 1, VNM_STRATEGY_DENSE_B = 2 };
int vnm_set_strategy(int strategy);
/* vnm_prepare with the operand form chosen for this one handle (DENSE_B falls back to GATHER where the form does
 * not exist).  The torch op asks for DENSE_B when its dense operand arrives as a transposed [N, K] view, which
 * only that form reads in place. */
int vnm_prepare_as(const void *values, const uint32_t *meta, const uint32_t *colloc,
                   int M, int K, int V, int n, int m, int strategy, vnm_handle_t *handle, void *stream);
int vnm_set_producer_warps(vnm_handle_t handle, int warps);
/* Dense-B form only: 1 (default) = products with at least one full wave of 512 x 240 tiles and M a multiple of 512 run on
 * pairs of SMs (thread-block clusters of two CTAs, tcgen05 cta_group::2: each CTA loads half of every B stage), 0 = always
 * the single-SM kernel, 2 = pairs without the L2 eviction-priority hints that ask the banded operand to stay cached,
 * 3 / 4 = pairs with one / two row tiles per CTA forced where the shape allows (default: two wherever 512-row tiles
 * fill the SM pairs, else one, whose two accumulators alternate between consecutive tiles).  Ablation switches; all
 * give identical bits. */
int vnm_set_pair_mode(vnm_handle_t handle, int mode);
/* Host-buffer entry points: number of equal column slices of the upload / product / download pipeline (1 .. 32; slices
 * are multiples of 256 columns and at least 1024 wide; 0 = the default, 8). */
int vnm_set_host_slices(vnm_handle_t handle, int slices);
/* Two-SM kernel: the producers also send L2-only prefetches (cp.async.bulk.prefetch) for the operands of the k-tile
 * `ktiles_ahead` further on (0 .. 32; 0 = none), beyond the three k-tiles the shared-memory rings hold.  Never changes a
 * result. */
int vnm_set_l2_prefetch(vnm_handle_t handle, int ktiles_ahead);
/* Caps the number of persistent CTAs (one per SM) the product of this handle launches; 0 = all SMs (default).  A caller
 * that runs something else beside the product (the multi-GPU launcher's all-gather, another stream's kernels) keeps SMs
 * free this way: a persistent CTA that has to wait for an SM would otherwise run after all the others.  No counterpart
 * in the reference (its kernels launch one CTA per tile). */
int vnm_set_max_ctas(vnm_handle_t handle, int max_ctas);
/* Shape and settings of a prepared operand (any output pointer may be NULL). */
int vnm_handle_info(vnm_handle_t handle, int *M, int *K, int *V, int *m, int *max_ctas);

/* Kernel configuration that vnm_spmm_f16 would launch for this handle and N (for reporting).  `stages`: for the dense-B
 * form 2 = the kernel on pairs of SMs, 1 = the one-SM kernel; for the gather form the number of producer warps. */
int vnm_spmm_config(vnm_handle_t handle, int N, int *tile_m, int *tile_n, int *stages, int *grid, int *smem_bytes);

/* ---------------------------------------------------------------------------------------------------------
 * Multi-GPU launcher: the dense operand and the result sharded by columns (N) over the GPUs of one node, the
 * sparse operand replicated.  One context per GPU (one process or host thread each, that GPU current).
 * The reference has no multi-GPU path (its harness and its torch op drive one GPU); these entry points are
 * what its callers would use in place of one vnm_prepare + vnm_spmm_f16 per process.
 * NCCL is loaded at run time (libnccl.so.2; a copy already loaded by the process is reused): VNM_ERR_UNSUPPORTED
 * if it cannot be found.  Collectives run on local buffers only.
 * --------------------------------------------------------------------------------------------------------- */
typedef struct vnm_mgpu_s *vnm_mgpu_t;
#define VNM_MGPU_ID_BYTES 128

/* Column range [lo, hi) of `rank`: contiguous, sizes differ by at most `multiple`, every boundary a multiple of
 * `multiple` (the product needs 8).  Pure arithmetic; needs neither a GPU nor NCCL. */
int vnm_mgpu_shard(int N, int world, int rank, int multiple, int *lo, int *hi);
/* Rank 0 fills VNM_MGPU_ID_BYTES bytes (an ncclUniqueId) and hands them to the other ranks by any means. */
int vnm_mgpu_unique_id(void *id128);
/* Joins the communicator on the CURRENT device (collective over all ranks: ncclCommInitRank, with NCCL kept to a few
 * CTAs because its kernels share the GPU with the product).  vnm_mgpu_create_from_comm adopts an ncclComm_t the caller
 * already has (it stays the caller's). */
int vnm_mgpu_create(const void *id128, int world, int rank, vnm_mgpu_t *ctx);
int vnm_mgpu_create_from_comm(void *nccl_comm, vnm_mgpu_t *ctx);
int vnm_mgpu_destroy(vnm_mgpu_t ctx);
int vnm_mgpu_info(vnm_mgpu_t ctx, int *world, int *rank);
/* SMs left free for NCCL's kernels while the chunks of a gathered product travel (default 16; 0 = none). */
int vnm_mgpu_set_comm_sms(vnm_mgpu_t ctx, int sms);
/* Replicates the three reference-format arrays from `root` (ncclBroadcast on `stream`); every rank passes buffers of
 * the sizes vnm_sizes gives, and then calls vnm_prepare on its copy. */
int vnm_mgpu_broadcast_operand(vnm_mgpu_t ctx, void *values, uint32_t *meta, uint32_t *colloc,
                               int M, int K, int V, int n, int m, int root, void *stream);
/* This rank's columns: exactly vnm_spmm_f16 on the shard -- the product has no exchange step. */
int vnm_mgpu_spmm_shard(vnm_mgpu_t ctx, vnm_handle_t handle, const void *B_shard, int64_t ldb, int n_shard,
                        const void *bias, void *out, int64_t ldo, int layout, void *stream);
/* The whole result on every rank: out_full is [N_total, M] fp16 (layout NM, ldo == M), rank r computes rows
 * [r * N_total / world, (r + 1) * N_total / world) from its B_shard [K, N_total / world] and receives the rest.
 * The shard is cut into `chunks` column chunks (clamped to 1..16 and to at least 256 columns each); chunk c+1 is
 * multiplied on `stream` while chunk c is exchanged on the context's second stream, each message landing at its final
 * rows.  chunks == 1 is the plain form: the product, then one in-place ncclAllGather.  `stream` continues after the last
 * chunk has arrived.  N_total must be a multiple of 8 x world. */
int vnm_mgpu_spmm_gathered(vnm_mgpu_t ctx, vnm_handle_t handle, const void *B_shard, int64_t ldb, int N_total,
                           const void *bias, void *out_full, int64_t ldo, int chunks, void *stream);

/* Peer-store form of the gathered product: no exchange step at all.  Every rank registers its [N_total, M] result
 * buffer once (collective: CUDA IPC handles of the allocation travel over the communicator and every peer's buffer is
 * mapped into this process; the buffer must come from cudaMalloc, e.g. a PyTorch tensor of the default allocator, and
 * all ranks must be processes on one node with peer access).  vnm_mgpu_spmm_gathered_p2p then runs ONE product launch
 * whose epilogue stores every output tile of this rank's rows to the same rows of all `world` buffers (its own first,
 * the peers' over NVLink), so the transfer of a tile overlaps the MMAs of the next ones; a small ncclAllGather on
 * `stream` before the launch (nobody still reads last call's result) and after it (every rank's rows have landed)
 * orders the ranks.  Needs world <= VNM_MAX_OUTS, ldo == M with M % 8 == 0, N_total % (8 x world) == 0;
 * VNM_ERR_UNSUPPORTED otherwise, and callers fall back to vnm_mgpu_spmm_gathered.  unregister is collective too: it
 * synchronises the device and the ranks before it unmaps, and returns only after every rank has unmapped, so the
 * buffer may be freed right after it. */
int vnm_mgpu_register_output(vnm_mgpu_t ctx, void *out_full, size_t bytes);
int vnm_mgpu_unregister_output(vnm_mgpu_t ctx, void *out_full);
int vnm_mgpu_spmm_gathered_p2p(vnm_mgpu_t ctx, vnm_handle_t handle, const void *B_shard, int64_t ldb, int N_total,
                               const void *bias, void *out_full, int64_t ldo, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* VENOM_B200_H_ */
