// Data-parallel gradient exchange: one NCCL communicator per context (one
// process per GPU), a single in-place sum all-reduce of the flat gradient
// bucket on the context's stream.  NCCL is resolved at run time with dlopen so
// that the library loads (and every single-GPU entry point works) on machines
// without it; a missing NCCL surfaces as KATSU_ERR_NCCL from these calls only.
//
// Small buckets (the low-channel layers' dW is a few KB) are latency-bound: NCCL's launch and
// protocol cost several tens of microseconds where the data needs one NVLink round trip.  For
// buckets up to 64 KiB the ranks of one machine therefore exchange through "mailboxes": every rank
// owns a small device buffer that the others map through CUDA IPC.  One kernel per rank copies its
// bucket into its own mailbox, raises a flag, waits (bounded) for the other ranks' flags and adds
// all mailboxes in rank order with plain peer loads, so every rank gets the same bits.  Larger
// buckets, ranks on several machines, or a machine without peer access use NCCL.
#include <dlfcn.h>
#include <string.h>
#include <unistd.h>

#include "common.cuh"

namespace {

// Minimal mirror of the NCCL declarations used here (stable since NCCL 2.x).
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;  // 0 == ncclSuccess
const int kNcclFloat32 = 7;
const int kNcclSum = 0;

struct NcclApi {
    void *handle;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t);
    const char *(*GetErrorString)(ncclResult_t);
};

NcclApi g_nccl = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};

int32_t load_nccl() {
    if (g_nccl.handle != nullptr) return KATSU_OK;
    // RTLD_NOLOAD first: reuse the copy a host framework already mapped.
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW);
    if (h == nullptr) return katsu_set_error(KATSU_ERR_NCCL, "libnccl.so.2 not found: %s", dlerror());
    NcclApi api;
    api.handle = h;
    api.GetUniqueId = (ncclResult_t(*)(ncclUniqueId *))dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (ncclResult_t(*)(ncclComm_t *, int, ncclUniqueId, int))dlsym(h, "ncclCommInitRank");
    api.CommDestroy = (ncclResult_t(*)(ncclComm_t))dlsym(h, "ncclCommDestroy");
    api.AllReduce = (ncclResult_t(*)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t))dlsym(
        h, "ncclAllReduce");
    api.AllGather = (ncclResult_t(*)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t))dlsym(h, "ncclAllGather");
    api.GetErrorString = (const char *(*)(ncclResult_t))dlsym(h, "ncclGetErrorString");
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.AllGather ||
        !api.GetErrorString)
        return katsu_set_error(KATSU_ERR_NCCL, "libnccl.so.2 lacks an expected symbol");
    g_nccl = api;
    return KATSU_OK;
}

int32_t nccl_fail(const char *what, ncclResult_t rc) {
    return katsu_set_error(KATSU_ERR_NCCL, "%s: %s", what, g_nccl.GetErrorString(rc));
}

// ---- mailbox all-reduce ---------------------------------------------------------------------
constexpr int kMaxRanks = 16;
constexpr size_t kMailFloats = 16384;                  // 64 KiB per slot
constexpr size_t kMailBytes = 2 * kMailFloats * 4 + 256;  // two slots, then two flags 128 bytes apart
constexpr long long kPeerWaitCycles = 2000000000ll;    // about a second of SM clocks

struct Mailboxes {
    float *box[kMaxRanks];   // box[rank] is this process's own allocation, the others are IPC mappings
    int ranks, rank;
    unsigned seq;            // calls so far; every rank makes the same calls in the same order
    bool enabled;
};

struct MailArgs {
    float *box[kMaxRanks];
    float *buf[kMaxRanks];   // buf[block]: the bucket this block reduces in place
    int ranks;               // ranks taking part in the sum
    int rank0;               // rank of block 0 (the self-test runs one block per emulated rank)
    unsigned seq;
    int count;
    int *status;
    long long budget;
};

#ifndef KATSU_EMU
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_relaxed_sys(const float *p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

// One block per rank (one block per process in production).  Slot = call parity: a rank cannot run
// two calls ahead of another one (its next call waits for that rank's flag of the same call), so
// the slot it overwrites has been read by everybody.
__global__ void __launch_bounds__(1024) mailbox_allreduce_kernel(MailArgs a) {
    const int rank = a.rank0 + (int)blockIdx.x;
    float *buf = a.buf[blockIdx.x];
    const unsigned slot = a.seq & 1u;
    float *mine = a.box[rank] + slot * kMailFloats;
    for (int i = threadIdx.x; i < a.count; i += blockDim.x) mine[i] = buf[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0)
        st_release_sys(reinterpret_cast<unsigned *>(a.box[rank] + 2 * kMailFloats) + slot * 32, a.seq);
    // lane r of the first warp waits for rank r's flag of this call, within the cycle budget
    __shared__ int arrived;
    if (threadIdx.x == 0) arrived = 0;
    __syncthreads();
    if ((int)threadIdx.x < a.ranks) {
        const unsigned *flag = reinterpret_cast<const unsigned *>(a.box[threadIdx.x] + 2 * kMailFloats) + slot * 32;
        const long long start = clock64();
        bool ok = false;
        for (unsigned poll = 0; poll < (1u << 26); ++poll) {
            if ((int)(ld_acquire_sys(flag) - a.seq) >= 0) { ok = true; break; }
            if ((poll & 63u) == 63u) {
                if (*reinterpret_cast<volatile int *>(a.status) != 0) break;  // another wait of this context gave up
                if (clock64() - start > a.budget) break;
            }
        }
        if (ok) atomicAdd(&arrived, 1);
    }
    __syncthreads();
    if (arrived != a.ranks) {
        if (threadIdx.x == 0) atomicCAS(a.status, 0, 31);  // a peer never showed up: results are undefined
        return;
    }
    for (int i = threadIdx.x; i < a.count; i += blockDim.x) {
        float sum = 0.f;
        for (int r = 0; r < a.ranks; ++r) sum += ld_relaxed_sys(a.box[r] + slot * kMailFloats + i);
        buf[i] = sum;
    }
}
#endif

// What the ranks tell each other while setting the mailboxes up.
struct MailHello {
    cudaIpcMemHandle_t handle;
    unsigned long long host;   // same value on every rank of one machine
    int ok;
    int pad;
};

unsigned long long host_identity() {
    // boot id of the machine (identical for every container on it); the host name as a fallback
    unsigned long long h = 1469598103934665603ull;
    char text[256] = {0};
    FILE *fh = fopen("/proc/sys/kernel/random/boot_id", "r");
    if (fh == nullptr || fgets(text, sizeof(text), fh) == nullptr) gethostname(text, sizeof(text) - 1);
    if (fh != nullptr) fclose(fh);
    for (const char *p = text; *p; ++p) h = (h ^ (unsigned char)*p) * 1099511628211ull;
    return h;
}

void mailboxes_release(katsu_cuda_ctx *ctx) {
    Mailboxes *mail = static_cast<Mailboxes *>(ctx->mailboxes);
    if (mail == nullptr) return;
    for (int r = 0; r < mail->ranks; ++r) {
        if (mail->box[r] == nullptr) continue;
        if (r == mail->rank)
            cudaFree(mail->box[r]);
        else
            cudaIpcCloseMemHandle(mail->box[r]);
    }
    cudaGetLastError();
    delete mail;
    ctx->mailboxes = nullptr;
}

// Collective over the communicator's ranks; every failure leaves NCCL as the only path (on all ranks).
void mailboxes_setup(katsu_cuda_ctx *ctx, int n_ranks, int rank) {
#ifndef KATSU_EMU
    if (n_ranks > kMaxRanks) return;
    Mailboxes *mail = new Mailboxes();
    memset(mail, 0, sizeof(*mail));
    mail->ranks = n_ranks;
    mail->rank = rank;
    ctx->mailboxes = mail;
    ncclComm_t comm = (ncclComm_t)ctx->comm;
    MailHello hello;
    memset(&hello, 0, sizeof(hello));
    hello.host = host_identity();
    void *own = nullptr;
    bool ok = cudaMalloc(&own, kMailBytes) == cudaSuccess && cudaMemset(own, 0, kMailBytes) == cudaSuccess;
    if (ok) mail->box[rank] = static_cast<float *>(own);
    if (ok && n_ranks > 1) ok = cudaIpcGetMemHandle(&hello.handle, own) == cudaSuccess;
    hello.ok = ok ? 1 : 0;
    cudaGetLastError();
    // exchange the handles (and whether everybody got this far) through the communicator itself
    MailHello *all = new MailHello[n_ranks];
    memset(all, 0, sizeof(MailHello) * n_ranks);
    void *dev = nullptr;
    bool exchanged = cudaMalloc(&dev, sizeof(MailHello) * (n_ranks + 1)) == cudaSuccess;
    if (exchanged) {
        char *send = static_cast<char *>(dev) + sizeof(MailHello) * n_ranks;
        exchanged = cudaMemcpyAsync(send, &hello, sizeof(hello), cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
                    g_nccl.AllGather(send, dev, sizeof(MailHello), 0 /* ncclInt8 */, comm, ctx->stream) == 0 &&
                    cudaMemcpyAsync(all, dev, sizeof(MailHello) * n_ranks, cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess &&
                    cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    }
    bool usable = exchanged;
    for (int r = 0; usable && r < n_ranks; ++r) usable = all[r].ok == 1 && all[r].host == hello.host;
    for (int r = 0; usable && r < n_ranks; ++r) {
        if (r == rank) continue;
        void *peer = nullptr;
        if (cudaIpcOpenMemHandle(&peer, all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            usable = false;
            break;
        }
        mail->box[r] = static_cast<float *>(peer);
    }
    cudaGetLastError();
    // second round: one rank that could not map a peer switches the path off for everybody
    if (exchanged) {
        float mine = usable ? 1.f : 0.f, total = 0.f;
        float *cell = static_cast<float *>(dev);
        const bool summed = cudaMemcpyAsync(cell, &mine, sizeof(float), cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
                            g_nccl.AllReduce(cell, cell, 1, kNcclFloat32, kNcclSum, comm, ctx->stream) == 0 &&
                            cudaMemcpyAsync(&total, cell, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess &&
                            cudaStreamSynchronize(ctx->stream) == cudaSuccess;
        usable = summed && total == float(n_ranks);
    }
    if (dev != nullptr) cudaFree(dev);
    delete[] all;
    cudaGetLastError();
    mail->enabled = usable;
    mail->seq = 0;
#else
    (void)ctx; (void)n_ranks; (void)rank;
#endif
}

}  // namespace

extern "C" int32_t katsu_cuda_comm_unique_id(uint8_t out_id[KATSU_COMM_ID_BYTES]) {
    KATSU_REQUIRE(out_id != nullptr, "out_id is null");
    KATSU_TRY(load_nccl());
    ncclUniqueId id;
    ncclResult_t rc = g_nccl.GetUniqueId(&id);
    if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
    static_assert(sizeof(id) == KATSU_COMM_ID_BYTES, "unique id size");
    memcpy(out_id, &id, sizeof(id));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_comm_init(katsu_cuda_ctx *ctx, const uint8_t id_bytes[KATSU_COMM_ID_BYTES],
                                        int32_t n_ranks, int32_t rank) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(id_bytes != nullptr, "id is null");
    KATSU_REQUIRE(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "bad rank / world size");
    KATSU_REQUIRE(ctx->comm == nullptr, "communicator already initialised");
    KATSU_TRY(load_nccl());
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof(id));
    ncclComm_t comm = nullptr;
    ncclResult_t rc = g_nccl.CommInitRank(&comm, n_ranks, id, rank);
    if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
    ctx->comm = comm;
    ctx->comm_ranks = n_ranks;
    ctx->comm_rank = rank;
    mailboxes_setup(ctx, n_ranks, rank);
    return KATSU_OK;
}

int32_t katsu_comm_destroy_impl(katsu_cuda_ctx *ctx) {
    Mailboxes *mail = static_cast<Mailboxes *>(ctx->mailboxes);
    if (mail != nullptr && mail->enabled && mail->ranks > 1 && ctx->comm != nullptr) {
        // A peer may still be reading this rank's mailbox in its last call.  One more collective
        // orders this point behind every rank's queued work; only then is the memory given back.
        float *cell = nullptr;
        if (cudaMalloc(&cell, sizeof(float)) == cudaSuccess) {
            cudaMemsetAsync(cell, 0, sizeof(float), ctx->stream);
            g_nccl.AllReduce(cell, cell, 1, kNcclFloat32, kNcclSum, (ncclComm_t)ctx->comm, ctx->stream);
            cudaStreamSynchronize(ctx->stream);
            cudaFree(cell);
        }
        cudaGetLastError();
    }
    mailboxes_release(ctx);
    if (ctx->comm != nullptr && g_nccl.handle != nullptr) g_nccl.CommDestroy((ncclComm_t)ctx->comm);
    ctx->comm = nullptr;
    ctx->comm_ranks = 0;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_comm_destroy(katsu_cuda_ctx *ctx) {
    KATSU_TRY(katsu_bind(ctx));
    cudaStreamSynchronize(ctx->stream);
    return katsu_comm_destroy_impl(ctx);
}

extern "C" int32_t katsu_cuda_allreduce_sum(katsu_cuda_ctx *ctx, float *buf, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(ctx->comm != nullptr, "no communicator: call katsu_cuda_comm_init first");
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(buf != nullptr, "buf is null");
#ifndef KATSU_EMU
    Mailboxes *mail = static_cast<Mailboxes *>(ctx->mailboxes);
    if (mail != nullptr && mail->enabled && count <= kMailFloats) {
        MailArgs args;
        memset(&args, 0, sizeof(args));
        for (int r = 0; r < mail->ranks; ++r) args.box[r] = mail->box[r];
        args.buf[0] = buf;
        args.ranks = mail->ranks;
        args.rank0 = mail->rank;
        args.seq = ++mail->seq;
        args.count = (int)count;
        args.status = ctx->status;
        args.budget = kPeerWaitCycles;
        KATSU_LAUNCH(ctx, mailbox_allreduce_kernel, 1, 1024, 0, args);
        return KATSU_OK;
    }
#endif
    ncclResult_t rc = g_nccl.AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, (ncclComm_t)ctx->comm, ctx->stream);
    if (rc != 0) return nccl_fail("ncclAllReduce", rc);
    return KATSU_OK;
}

// Diagnostic: the mailbox all-reduce with `ranks` emulated ranks on this one device, one block each
// in a cooperative launch (the blocks wait on one another, so they must be resident together).
// buf holds ranks * count floats, rank r's bucket at r * count; afterwards every bucket holds the
// sum.  With absent > 0 the last `absent` ranks never run: the others give up after `cycles` SM
// clocks, the kernel returns and the next synchronising call reports KATSU_ERR_TIMEOUT -- the path a
// rank takes when a peer process has died, exercised without a second process or a fault.
extern "C" int32_t katsu_cuda_selftest_mailbox_allreduce(katsu_cuda_ctx *ctx, float *buf, int32_t ranks, size_t count,
                                                         int32_t absent, uint64_t cycles) {
    KATSU_TRY(katsu_bind(ctx));
#ifndef KATSU_EMU
    KATSU_REQUIRE(buf != nullptr && ranks >= 1 && ranks <= kMaxRanks && absent >= 0 && absent < ranks, "bad rank counts");
    KATSU_REQUIRE(count >= 1 && count <= kMailFloats, "count outside the mailbox size");
    KATSU_REQUIRE(cycles >= 1000 && cycles <= 2000000000ull, "cycle budget must be between 1e3 and 2e9");
    void *boxes = nullptr;
    KATSU_TRY(katsu_pool_alloc(ctx, kMailBytes * ranks, &boxes));
    int32_t rc = KATSU_OK;
    if (cudaMemsetAsync(boxes, 0, kMailBytes * ranks, ctx->stream) != cudaSuccess)
        rc = katsu_set_error(KATSU_ERR_CUDA, "cudaMemsetAsync failed (mailbox self-test)");
    MailArgs args;
    memset(&args, 0, sizeof(args));
    for (int r = 0; r < ranks; ++r) {
        args.box[r] = reinterpret_cast<float *>(static_cast<char *>(boxes) + kMailBytes * r);
        args.buf[r] = buf + size_t(r) * count;
    }
    args.ranks = ranks;
    args.rank0 = 0;
    args.seq = 1;
    args.count = (int)count;
    args.status = ctx->status;
    args.budget = (long long)cycles;
    if (rc == KATSU_OK) {
        void *params[] = {&args};
        cudaError_t err = cudaLaunchCooperativeKernel((const void *)mailbox_allreduce_kernel, dim3(ranks - absent), dim3(1024),
                                                      params, 0, ctx->stream);
        ctx->launches += 1;
        if (err != cudaSuccess) rc = katsu_set_error(KATSU_ERR_CUDA, "cooperative launch failed: %s", cudaGetErrorString(err));
    }
    cudaFreeAsync(boxes, ctx->stream);
    return rc;
#else
    (void)buf; (void)ranks; (void)count; (void)absent; (void)cycles;
    return katsu_set_error(KATSU_ERR_UNSUPPORTED, "not available in this build");
#endif
}
