// vnm_mgpu_*: the N-sharded multi-GPU launcher behind the C ABI (one process, or one host thread, per GPU).
//
// Column c of C = A * B depends only on column c of B, so the dense operand and the result are split by columns
// across the ranks and the sparse operand is replicated (vnm_mgpu_broadcast_operand, once).  The product itself
// needs no communication (vnm_mgpu_spmm_shard).  Only a caller that needs the whole [N, M] result on every rank
// asks for vnm_mgpu_spmm_gathered, which overlaps the exchange with the product: the shard is cut into column
// chunks, chunk c+1 is multiplied while chunk c travels on a second stream, each rank writing and receiving
// straight into the final [N, M] buffer (an N-shard is a contiguous block of its rows).  While chunks travel the
// product runs with a few SMs left free, because NCCL's kernels need SMs of their own and a persistent CTA that
// had to wait for one would run after all the others.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, preferring a copy the process has already loaded, e.g.
// PyTorch's): the library has no link-time dependency on it and single-GPU users never load it.
//
// vnm_mgpu_spmm_gathered_p2p is the form without an exchange step: result buffers registered through CUDA IPC are
// mapped into every rank, and the product's epilogue stores each output tile to all of them with plain (non-multicast)
// TMA stores, its own buffer first and the peers' over NVLink.  No kernel of this library READS a peer's memory, and
// ranks wait for one another only in NCCL collectives, never inside a kernel of this library.
#include "../../include/venom_b200.h"
#include "vnm_internal.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

using namespace vnm;

namespace {

int mfail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    return set_last_error(code, buf);
}

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommCount)(const ncclComm_t, int *);
    ncclResult_t (*CommUserRank)(const ncclComm_t, int *);
    ncclResult_t (*CommCuDevice)(const ncclComm_t, int *);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    const char *(*GetErrorString)(ncclResult_t);
    bool ok = false;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

template <typename F>
bool bind(void *lib, const char *name, F *fn, bool required = true)
{
    *fn = reinterpret_cast<F>(dlsym(lib, name));
    return *fn != nullptr || !required;
}

const NcclApi *nccl()
{
    std::call_once(g_nccl_once, [] {
        void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // a copy the process already uses, if any
        if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) return;
        NcclApi &a = g_nccl;
        bool ok = bind(lib, "ncclGetUniqueId", &a.GetUniqueId) && bind(lib, "ncclCommInitRank", &a.CommInitRank) &&
                  bind(lib, "ncclCommInitRankConfig", &a.CommInitRankConfig, false) && bind(lib, "ncclCommDestroy", &a.CommDestroy) &&
                  bind(lib, "ncclCommCount", &a.CommCount) && bind(lib, "ncclCommUserRank", &a.CommUserRank) &&
                  bind(lib, "ncclCommCuDevice", &a.CommCuDevice) && bind(lib, "ncclGroupStart", &a.GroupStart) &&
                  bind(lib, "ncclGroupEnd", &a.GroupEnd) && bind(lib, "ncclBroadcast", &a.Broadcast) &&
                  bind(lib, "ncclAllGather", &a.AllGather) && bind(lib, "ncclSend", &a.Send) && bind(lib, "ncclRecv", &a.Recv) &&
                  bind(lib, "ncclGetErrorString", &a.GetErrorString);
        a.ok = ok;
    });
    return g_nccl.ok ? &g_nccl : nullptr;
}

#define VNM_NCCL(call, what)                                                                                   \
    do {                                                                                                       \
        ncclResult_t r__ = (call);                                                                             \
        if (r__ != ncclSuccess) return mfail(VNM_ERR_CUDA, "%s: NCCL error %d (%s)", what, (int)r__, api->GetErrorString(r__)); \
    } while (0)
#define VNM_CU(call, what)                                                                        \
    do {                                                                                          \
        cudaError_t e__ = (call);                                                                 \
        if (e__ != cudaSuccess) return mfail(VNM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e__)); \
    } while (0)

constexpr int kMaxChunks = 16;

// what a rank tells the others about a result buffer: the IPC handle of the allocation that holds it and where in
// that allocation the buffer starts
struct IpcNote {
    cudaIpcMemHandle_t handle;
    unsigned long long offset, bytes;
    int ok, device;
};

struct PeerMapping {      // one opened allocation of one peer (an allocation may hold several registered buffers)
    int rank;
    cudaIpcMemHandle_t handle;
    void *base;
    int refs;
};

struct Registered {
    void *local;
    size_t bytes;
    void *peer[MAX_OUTS];  // [rank] the buffer of that rank in this process's address space (own rank: local)
};

typedef CUresult (*AddressRangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
AddressRangeFn get_address_range_fn()
{
    static AddressRangeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (AddressRangeFn)p;
    });
    return fn;
}

}  // namespace

struct vnm_mgpu_s {
    ncclComm_t comm;
    bool owns_comm;
    int world, rank, device;
    int comm_sms;              // SMs left to NCCL while chunks of a gathered product travel
    cudaStream_t comm_stream;  // the exchange runs here, beside the product on the caller's stream
    cudaEvent_t chunk_done[kMaxChunks];
    cudaEvent_t joined;
    IpcNote *notes;            // device: [world] exchange buffer of register_output
    int *sync_words;           // device: [world] payload of the small all-gathers that order the ranks around a peer-store product
    std::vector<PeerMapping> mappings;
    std::vector<Registered> registered;
};

extern "C" {

int vnm_mgpu_shard(int N, int world, int rank, int multiple, int *lo, int *hi)
{
    if (N <= 0 || world <= 0 || rank < 0 || rank >= world || multiple <= 0 || !lo || !hi)
        return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_shard: bad arguments (N=%d world=%d rank=%d multiple=%d)", N, world, rank, multiple);
    if (N % multiple) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_shard: N (%d) must be a multiple of %d", N, multiple);
    const int units = N / multiple, base = units / world, extra = units % world;
    const int l = rank * base + (rank < extra ? rank : extra);
    *lo = l * multiple;
    *hi = (l + base + (rank < extra ? 1 : 0)) * multiple;
    return VNM_OK;
}

int vnm_mgpu_unique_id(void *id128)
{
    if (!id128) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_unique_id: null pointer");
    const NcclApi *api = nccl();
    if (!api) return mfail(VNM_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded: %s", dlerror() ? dlerror() : "missing symbols");
    static_assert(sizeof(ncclUniqueId) == VNM_MGPU_ID_BYTES, "unique id size");
    VNM_NCCL(api->GetUniqueId(reinterpret_cast<ncclUniqueId *>(id128)), "ncclGetUniqueId");
    return VNM_OK;
}

static int finish_create(vnm_mgpu_s *c, vnm_mgpu_t *ctx)
{
    // highest priority: when a chunk's exchange and the next chunk's product become runnable together, NCCL's few CTAs
    // are placed first and the product fills the SMs that remain
    int prio_low = 0, prio_high = 0;
    cudaError_t e = cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high);
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&c->comm_stream, cudaStreamNonBlocking, prio_high);
    for (int i = 0; e == cudaSuccess && i < kMaxChunks; i++) e = cudaEventCreateWithFlags(&c->chunk_done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->joined, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaMalloc(&c->notes, sizeof(IpcNote) * (size_t)c->world);
    if (e == cudaSuccess) e = cudaMalloc(&c->sync_words, sizeof(int) * (size_t)c->world);
    if (e == cudaSuccess) e = cudaMemset(c->sync_words, 0, sizeof(int) * (size_t)c->world);
    if (e != cudaSuccess) {
        vnm_mgpu_destroy(c);
        return mfail(VNM_ERR_CUDA, "vnm_mgpu_create: %s", cudaGetErrorString(e));
    }
    *ctx = c;
    return VNM_OK;
}

int vnm_mgpu_create(const void *id128, int world, int rank, vnm_mgpu_t *ctx)
{
    if (!id128 || !ctx || world <= 0 || rank < 0 || rank >= world) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_create: bad arguments");
    const NcclApi *api = nccl();
    if (!api) return mfail(VNM_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    vnm_mgpu_s *c = new (std::nothrow) vnm_mgpu_s();
    if (!c) return mfail(VNM_ERR_CUDA, "out of host memory");
    c->world = world; c->rank = rank; c->owns_comm = true; c->comm_sms = 16;
    VNM_CU(cudaGetDevice(&c->device), "cudaGetDevice");
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclResult_t r;
    if (api->CommInitRankConfig) {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.maxCTAs = c->comm_sms;  // the exchange shares the GPU with the product: keep its footprint to the SMs left free
        r = api->CommInitRankConfig(&c->comm, world, id, rank, &cfg);
    } else {
        r = api->CommInitRank(&c->comm, world, id, rank);
    }
    if (r != ncclSuccess) {
        delete c;
        return mfail(VNM_ERR_CUDA, "ncclCommInitRank: NCCL error %d (%s)", (int)r, api->GetErrorString(r));
    }
    return finish_create(c, ctx);
}

int vnm_mgpu_create_from_comm(void *nccl_comm, vnm_mgpu_t *ctx)
{
    if (!nccl_comm || !ctx) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_create_from_comm: null pointer");
    const NcclApi *api = nccl();
    if (!api) return mfail(VNM_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    vnm_mgpu_s *c = new (std::nothrow) vnm_mgpu_s();
    if (!c) return mfail(VNM_ERR_CUDA, "out of host memory");
    c->comm = (ncclComm_t)nccl_comm;
    c->owns_comm = false;
    c->comm_sms = 32;  // an adopted communicator keeps whatever channel count its owner configured
    VNM_NCCL(api->CommCount(c->comm, &c->world), "ncclCommCount");
    VNM_NCCL(api->CommUserRank(c->comm, &c->rank), "ncclCommUserRank");
    VNM_NCCL(api->CommCuDevice(c->comm, &c->device), "ncclCommCuDevice");
    return finish_create(c, ctx);
}

int vnm_mgpu_destroy(vnm_mgpu_t c)
{
    if (!c) return VNM_OK;
    if (c->comm_stream) cudaStreamSynchronize(c->comm_stream);
    if (!c->mappings.empty()) {
        // peers' buffers still mapped: the caller should have unregistered (collectively); unmap after this device is idle
        cudaDeviceSynchronize();
        for (PeerMapping &m : c->mappings) cudaIpcCloseMemHandle(m.base);
        c->mappings.clear();
    }
    if (c->notes) cudaFree(c->notes);
    if (c->sync_words) cudaFree(c->sync_words);
    for (cudaEvent_t e : c->chunk_done)
        if (e) cudaEventDestroy(e);
    if (c->joined) cudaEventDestroy(c->joined);
    if (c->comm_stream) cudaStreamDestroy(c->comm_stream);
    if (c->owns_comm && c->comm && nccl()) nccl()->CommDestroy(c->comm);
    delete c;
    return VNM_OK;
}

int vnm_mgpu_info(vnm_mgpu_t c, int *world, int *rank)
{
    if (!c) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_info: null context");
    if (world) *world = c->world;
    if (rank) *rank = c->rank;
    return VNM_OK;
}

int vnm_mgpu_set_comm_sms(vnm_mgpu_t c, int sms)
{
    if (!c || sms < 0 || sms > 64) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_set_comm_sms: need a context and 0 <= sms <= 64");
    c->comm_sms = sms;
    return VNM_OK;
}

int vnm_mgpu_broadcast_operand(vnm_mgpu_t c, void *values, uint32_t *meta, uint32_t *colloc, int M, int K, int V, int n, int m, int root,
                               void *stream)
{
    if (!c || !values || !meta || !colloc) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_broadcast_operand: null pointer");
    if (root < 0 || root >= c->world) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_broadcast_operand: root %d outside the communicator", root);
    int64_t nv = 0, nm = 0, nc = 0;
    if (int rc = vnm_sizes(M, K, V, n, m, nullptr, &nv, &nm, &nc)) return rc;
    const NcclApi *api = nccl();
    cudaStream_t s = (cudaStream_t)stream;
    VNM_NCCL(api->GroupStart(), "ncclGroupStart");
    VNM_NCCL(api->Broadcast(values, values, (size_t)nv * 2, ncclChar, root, c->comm, s), "ncclBroadcast(values)");
    VNM_NCCL(api->Broadcast(meta, meta, (size_t)nm * 4, ncclChar, root, c->comm, s), "ncclBroadcast(metadata)");
    VNM_NCCL(api->Broadcast(colloc, colloc, (size_t)nc * 4, ncclChar, root, c->comm, s), "ncclBroadcast(column-loc)");
    VNM_NCCL(api->GroupEnd(), "ncclGroupEnd");
    return VNM_OK;
}

int vnm_mgpu_spmm_shard(vnm_mgpu_t c, vnm_handle_t h, const void *B_shard, int64_t ldb, int n_shard, const void *bias, void *out, int64_t ldo,
                        int layout, void *stream)
{
    if (!c) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_spmm_shard: null context");
    return vnm_spmm_f16(h, B_shard, ldb, n_shard, bias, out, ldo, layout, stream);  // no communication: columns are independent
}

int vnm_mgpu_spmm_gathered(vnm_mgpu_t c, vnm_handle_t h, const void *B_shard, int64_t ldb, int N_total, const void *bias, void *out_full,
                           int64_t ldo, int chunks, void *stream)
{
    if (!c || !h || !B_shard || !out_full) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_spmm_gathered: null pointer");
    const int W = c->world;
    if (N_total <= 0 || N_total % (8 * W) != 0)
        return mfail(VNM_ERR_UNSUPPORTED, "vnm_mgpu_spmm_gathered: N (%d) must be a multiple of 8 x ranks (%d) so that every rank holds the same number of columns",
                     N_total, 8 * W);
    int M = 0, user_cap = 0;
    if (int rc = vnm_handle_info(h, &M, nullptr, nullptr, nullptr, &user_cap)) return rc;
    if (ldo != M)
        return mfail(VNM_ERR_UNSUPPORTED, "vnm_mgpu_spmm_gathered: the gathered [N, M] result must be dense (ldo == M = %d, got %lld): whole row "
                     "blocks travel as single messages", M, (long long)ldo);
    const NcclApi *api = nccl();
    if (!api) return mfail(VNM_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    const int ns = N_total / W;  // columns per rank = rows of the [N, M] result per rank
    if (chunks < 1) chunks = 1;
    if (chunks > kMaxChunks) chunks = kMaxChunks;
    // chunk width: a multiple of 8 columns; never so small that launch overheads dominate
    int w = ((ns + chunks - 1) / chunks + 7) / 8 * 8;
    if (w < 256) w = ns < 256 ? ns : 256;
    chunks = (ns + w - 1) / w;
    cudaStream_t s = (cudaStream_t)stream;
    __half *out = (__half *)out_full;
    const bool overlap = W > 1 && chunks > 1;
    if (overlap && c->comm_sms > 0) {
        int sms = 0;
        VNM_CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device), "cudaDeviceGetAttribute");
        int cap = sms > c->comm_sms + 8 ? sms - c->comm_sms : 0;
        if (user_cap > 0 && (cap == 0 || user_cap < cap)) cap = user_cap;
        if (int rc = vnm_set_max_ctas(h, cap)) return rc;
    }
    int rc = VNM_OK;
    for (int ch = 0; ch < chunks && rc == VNM_OK; ++ch) {
        const int c0 = ch * w, cw = ns - c0 < w ? ns - c0 : w;
        __half *mine = out + ((int64_t)c->rank * ns + c0) * ldo;
        rc = vnm_spmm_f16(h, (const __half *)B_shard + c0, ldb, cw, bias, mine, ldo, VNM_LAYOUT_NM, s);
        if (rc != VNM_OK || W == 1) continue;
        // chunk ch is final on `s`: exchange it on the second stream while the next chunk is multiplied
        cudaStream_t xs = overlap ? c->comm_stream : s;
        if (overlap) {
            VNM_CU(cudaEventRecord(c->chunk_done[ch], s), "cudaEventRecord");
            VNM_CU(cudaStreamWaitEvent(c->comm_stream, c->chunk_done[ch], 0), "cudaStreamWaitEvent");
        }
        if (chunks == 1) {
            // whole shards, rows contiguous: one in-place all-gather (rank r's block already sits at r * ns)
            VNM_NCCL(api->AllGather(mine, out, (size_t)ns * M * 2, ncclChar, c->comm, xs), "ncclAllGather");
        } else {
            // every rank sends its chunk to every peer and receives the peers' chunks at their final rows
            VNM_NCCL(api->GroupStart(), "ncclGroupStart");
            for (int r = 0; r < W; ++r) {
                if (r == c->rank) continue;
                __half *theirs = out + ((int64_t)r * ns + c0) * ldo;
                VNM_NCCL(api->Send(mine, (size_t)cw * M * 2, ncclChar, r, c->comm, xs), "ncclSend");
                VNM_NCCL(api->Recv(theirs, (size_t)cw * M * 2, ncclChar, r, c->comm, xs), "ncclRecv");
            }
            VNM_NCCL(api->GroupEnd(), "ncclGroupEnd");
        }
    }
    if (overlap) {
        // the caller's stream continues only after the last chunk has arrived everywhere
        cudaEventRecord(c->joined, c->comm_stream);
        cudaStreamWaitEvent(s, c->joined, 0);
        vnm_set_max_ctas(h, user_cap);
    }
    return rc;
}

// A small all-gather on `s`: returns (in stream order) on a rank only after every rank has reached the same point.
static int rank_barrier(vnm_mgpu_s *c, const NcclApi *api, cudaStream_t s)
{
    VNM_NCCL(api->AllGather(c->sync_words + c->rank, c->sync_words, sizeof(int), ncclChar, c->comm, s), "ncclAllGather (rank barrier)");
    return VNM_OK;
}

static void release_mapping(vnm_mgpu_s *c, int rank, void *peer_ptr)
{
    for (size_t i = 0; i < c->mappings.size(); ++i) {
        PeerMapping &m = c->mappings[i];
        if (m.rank != rank || (char *)peer_ptr < (char *)m.base) continue;
        // the mapping that holds peer_ptr: the one with the closest base below it
        bool closest = true;
        for (const PeerMapping &o : c->mappings)
            if (o.rank == rank && (char *)o.base > (char *)m.base && (char *)o.base <= (char *)peer_ptr) closest = false;
        if (!closest) continue;
        if (--m.refs == 0) {
            cudaIpcCloseMemHandle(m.base);
            c->mappings.erase(c->mappings.begin() + (long)i);
        }
        return;
    }
}

int vnm_mgpu_register_output(vnm_mgpu_t c, void *out_full, size_t bytes)
{
    if (!c || !out_full || bytes == 0) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_register_output: null pointer or empty buffer");
    const NcclApi *api = nccl();
    if (!api) return mfail(VNM_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    const int W = c->world;
    for (const Registered &r : c->registered)
        if (r.local == out_full) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_register_output: this buffer is already registered");
    // every rank takes part in both exchanges below even if something failed locally, so that nobody waits forever
    IpcNote mine;
    memset(&mine, 0, sizeof(mine));
    mine.device = c->device;
    char why[256] = "";
    if (W > MAX_OUTS) {
        snprintf(why, sizeof(why), "at most %d ranks", MAX_OUTS);
    } else {
        AddressRangeFn range = get_address_range_fn();
        CUdeviceptr base = 0;
        size_t span = 0;
        if (!range || range(&base, &span, (CUdeviceptr)out_full) != CUDA_SUCCESS) {
            snprintf(why, sizeof(why), "the buffer is not inside a device allocation of this process");
        } else if ((size_t)((char *)out_full - (char *)base) + bytes > span) {
            snprintf(why, sizeof(why), "the buffer runs past the end of its allocation");
        } else {
            cudaError_t e = cudaIpcGetMemHandle(&mine.handle, (void *)base);
            if (e != cudaSuccess) {
                snprintf(why, sizeof(why), "cudaIpcGetMemHandle: %s (the buffer must come from cudaMalloc)", cudaGetErrorString(e));
                cudaGetLastError();
            } else {
                mine.offset = (unsigned long long)((char *)out_full - (char *)base);
                mine.bytes = bytes;
                mine.ok = 1;
            }
        }
    }
    std::vector<IpcNote> all((size_t)W);
    cudaStream_t xs = c->comm_stream;
    VNM_CU(cudaMemcpyAsync(c->notes + c->rank, &mine, sizeof(mine), cudaMemcpyHostToDevice, xs), "cudaMemcpyAsync");
    VNM_NCCL(api->AllGather(c->notes + c->rank, c->notes, sizeof(IpcNote), ncclChar, c->comm, xs), "ncclAllGather (IPC handles)");
    VNM_CU(cudaMemcpyAsync(all.data(), c->notes, sizeof(IpcNote) * (size_t)W, cudaMemcpyDeviceToHost, xs), "cudaMemcpyAsync");
    VNM_CU(cudaStreamSynchronize(xs), "cudaStreamSynchronize");
    bool everyone = true;
    for (int r = 0; r < W; ++r) everyone = everyone && all[(size_t)r].ok && all[(size_t)r].bytes == bytes;
    Registered reg;
    memset(&reg, 0, sizeof(reg));
    reg.local = out_full;
    reg.bytes = bytes;
    int opened_ok = everyone ? 1 : 0;
    if (everyone) {
        for (int r = 0; r < W && opened_ok; ++r) {
            if (r == c->rank) { reg.peer[r] = out_full; continue; }
            const IpcNote &n = all[(size_t)r];
            if (n.device == c->device) {
                snprintf(why, sizeof(why), "rank %d uses the same device", r);
                opened_ok = 0;
                break;
            }
            PeerMapping *have = nullptr;
            for (PeerMapping &m : c->mappings)
                if (m.rank == r && memcmp(&m.handle, &n.handle, sizeof(n.handle)) == 0) have = &m;
            if (!have) {
                void *base = nullptr;
                cudaError_t e = cudaIpcOpenMemHandle(&base, n.handle, cudaIpcMemLazyEnablePeerAccess);
                if (e != cudaSuccess) {
                    snprintf(why, sizeof(why), "cudaIpcOpenMemHandle (rank %d): %s", r, cudaGetErrorString(e));
                    cudaGetLastError();
                    opened_ok = 0;
                    break;
                }
                PeerMapping m;
                m.rank = r; m.handle = n.handle; m.base = base; m.refs = 0;
                c->mappings.push_back(m);
                have = &c->mappings.back();
            }
            have->refs++;
            reg.peer[r] = (char *)have->base + n.offset;
        }
    }
    // second round: did every rank map every peer?
    IpcNote verdict;
    memset(&verdict, 0, sizeof(verdict));
    verdict.ok = opened_ok;
    VNM_CU(cudaMemcpyAsync(c->notes + c->rank, &verdict, sizeof(verdict), cudaMemcpyHostToDevice, xs), "cudaMemcpyAsync");
    VNM_NCCL(api->AllGather(c->notes + c->rank, c->notes, sizeof(IpcNote), ncclChar, c->comm, xs), "ncclAllGather (IPC verdict)");
    VNM_CU(cudaMemcpyAsync(all.data(), c->notes, sizeof(IpcNote) * (size_t)W, cudaMemcpyDeviceToHost, xs), "cudaMemcpyAsync");
    VNM_CU(cudaStreamSynchronize(xs), "cudaStreamSynchronize");
    bool all_ok = true;
    for (int r = 0; r < W; ++r) all_ok = all_ok && all[(size_t)r].ok;
    if (!all_ok) {
        for (int r = 0; r < W; ++r)
            if (r != c->rank && reg.peer[r]) release_mapping(c, r, reg.peer[r]);
        return mfail(VNM_ERR_UNSUPPORTED, "vnm_mgpu_register_output: the result buffers could not be shared between the ranks%s%s", why[0] ? ": " : " (another rank failed)",
                     why);
    }
    c->registered.push_back(reg);
    return VNM_OK;
}

int vnm_mgpu_unregister_output(vnm_mgpu_t c, void *out_full)
{
    if (!c || !out_full) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_unregister_output: null pointer");
    const NcclApi *api = nccl();
    if (!api) return mfail(VNM_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    size_t at = c->registered.size();
    for (size_t i = 0; i < c->registered.size(); ++i)
        if (c->registered[i].local == out_full) at = i;
    if (at == c->registered.size()) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_unregister_output: this buffer is not registered");
    // nobody may still be storing into a buffer that is about to be unmapped: all work of this device, then all ranks
    VNM_CU(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (int rc = rank_barrier(c, api, c->comm_stream)) return rc;
    VNM_CU(cudaStreamSynchronize(c->comm_stream), "cudaStreamSynchronize");
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank) release_mapping(c, r, c->registered[at].peer[r]);
    c->registered.erase(c->registered.begin() + (long)at);
    // and nobody may free its buffer while a peer still has it mapped: return only after every rank has unmapped
    if (int rc = rank_barrier(c, api, c->comm_stream)) return rc;
    VNM_CU(cudaStreamSynchronize(c->comm_stream), "cudaStreamSynchronize");
    return VNM_OK;
}

int vnm_mgpu_spmm_gathered_p2p(vnm_mgpu_t c, vnm_handle_t h, const void *B_shard, int64_t ldb, int N_total, const void *bias, void *out_full,
                               int64_t ldo, void *stream)
{
    if (!c || !h || !B_shard || !out_full) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_spmm_gathered_p2p: null pointer");
    const int W = c->world;
    if (W > MAX_OUTS) return mfail(VNM_ERR_UNSUPPORTED, "vnm_mgpu_spmm_gathered_p2p: at most %d ranks", MAX_OUTS);
    if (N_total <= 0 || N_total % (8 * W) != 0)
        return mfail(VNM_ERR_UNSUPPORTED, "vnm_mgpu_spmm_gathered_p2p: N (%d) must be a multiple of 8 x ranks (%d)", N_total, 8 * W);
    int M = 0;
    if (int rc = vnm_handle_info(h, &M, nullptr, nullptr, nullptr, nullptr)) return rc;
    if (ldo != M) return mfail(VNM_ERR_UNSUPPORTED, "vnm_mgpu_spmm_gathered_p2p: the gathered [N, M] result must be dense (ldo == M = %d, got %lld)", M, (long long)ldo);
    const Registered *reg = nullptr;
    for (const Registered &r : c->registered)
        if (r.local == out_full) reg = &r;
    if (!reg) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_spmm_gathered_p2p: out_full was not registered with vnm_mgpu_register_output");
    if ((size_t)N_total * (size_t)M * 2 > reg->bytes) return mfail(VNM_ERR_BAD_ARG, "vnm_mgpu_spmm_gathered_p2p: the registered buffer is smaller than [N, M]");
    const NcclApi *api = nccl();
    if (!api) return mfail(VNM_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    cudaStream_t s = (cudaStream_t)stream;
    const int ns = N_total / W;
    const size_t row0 = (size_t)c->rank * (size_t)ns * (size_t)ldo * 2;  // byte offset of this rank's rows in every buffer
    void *outs[MAX_OUTS];
    for (int i = 0; i < W; ++i) outs[i] = (char *)reg->peer[(c->rank + i) % W] + row0;  // own buffer first, then the peers in ring order
    if (W > 1)
        if (int rc = rank_barrier(c, api, s)) return rc;   // nobody still reads the previous contents of any buffer
    int rc = vnm_spmm_f16_multi(h, B_shard, ldb, ns, bias, outs, W, ldo, VNM_LAYOUT_NM, s);
    // the closing barrier is issued even after a failed launch: the other ranks are going to wait in theirs
    if (W > 1) {
        int rb = rank_barrier(c, api, s);                   // every rank's rows have landed everywhere
        if (rc == VNM_OK) rc = rb;
    }
    return rc;
}

}  // extern "C"
