// Thin inline-PTX layer for the Blackwell (sm_100a) data path used by the
// tensor-core kernels: mbarrier, TMA tiled loads, tcgen05 MMA / commit / TMEM
// allocation and loads, plus the shared-memory and instruction descriptors.
//
// Every wait is bounded: a wait that runs out records a code in the context's
// status word and returns false, and callers fall through to their normal
// teardown (TMEM freed, kernel returns), so a logic error cannot hang the GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .b32 rx;\n"
        ".reg .pred px;\n"
        "elect.sync rx|px, 0xFFFFFFFF;\n"
        "selp.u32 %0, 1, 0, px;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// Shared-memory stores through the shared window.  Pointers derived from the manually
// aligned dynamic shared-memory base are generic to the compiler, and generic stores that
// land in shared memory were measured ~7x slower than st.shared on this part.
__device__ __forceinline__ void st_shared_f32(void *p, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_u32(p)), "f"(v) : "memory");
}

__device__ __forceinline__ float ld_shared_f32(const void *p) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}

__device__ __forceinline__ float4 ld_shared_v4(const void *p) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(p)) : "memory");
    return v;
}

__device__ __forceinline__ void st_shared_v4(void *p, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(smem_u32(p)), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One poll (the hardware may park the thread for a short, implementation-defined time).
// Measured: an explicit suspend-time hint of 100 us made the pipelined stem kernels 3-5 %
// slower, so none is given.
// One arrival for the whole warp, after every lane has finished what the barrier guards.
// 32 lanes arriving on one barrier are 32 serialised shared-memory operations; the pipelined
// stem kernels hand off every few hundred cycles, where that was a large share of the
// shared-memory pipe's time.  Barriers used this way are initialised with a count of warps.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t *bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait: gives up after about a second of SM clocks (and never more
// than kWaitPolls polls).  On expiry: status word := code (first failure
// wins) and false is returned.
constexpr uint32_t kWaitPolls = 1u << 24;
constexpr long long kWaitCycles = 2000000000ll;

__device__ __forceinline__ bool mbar_wait_budget(uint64_t *bar, uint32_t parity, int *status, int code,
                                                 long long cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t i = 0; i < kWaitPolls; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            // once any wait of the launch has given up, the others follow at once instead of
            // each running out its own budget
            if (status != nullptr && *reinterpret_cast<volatile int *>(status) != 0) return false;
            if (clock64() - start > cycles) break;
        }
    }
    if (status != nullptr) atomicCAS(status, 0, code);
    return false;
}

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *status, int code) {
    return mbar_wait_budget(bar, parity, status, code, kWaitCycles);
}

// Whole-warp wait for a barrier that is usually NOT yet complete: lane 0 polls, the warp then
// reconverges.  32 lanes re-polling one barrier are 32 shared-memory operations per poll,
// enough to starve the shared-memory pipe of a block whose other warps are storing tiles.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, int *status, int code) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, status, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);  // also orders lane 0's acquire before the other lanes' accesses
    return ok != 0;
}

// Whole-warp wait for a barrier that is usually ALREADY complete (an MMA-issue warp whose
// producers run ahead).  Every lane polls once and the warp votes, so it stays converged.
// Measured in an MMA-issue loop: a wait on a completed barrier costs ~90
// cycles this way and ~220 when lane 0 polls inside a divergent region, because the warp
// leaves and re-enters uniform control flow.  Falls back to mbar_wait_warp when not ready.
__device__ __forceinline__ bool mbar_wait_warp_ready(uint64_t *bar, uint32_t parity, int *status, int code) {
    // The vote makes the decision warp-uniform: the phase may complete between two lanes'
    // polls, and lanes that disagreed would meet different warp-level instructions next.
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity) ? 1 : 0)) return true;
    return mbar_wait_warp(bar, parity, status, code);
}

// Orders this thread's generic-proxy accesses to shared memory (ld.shared / st.shared) against later
// async-proxy accesses (tcgen05.mma operand reads, TMA loads and stores).  Needed in both directions:
//  * after st.shared into a tile that tcgen05.mma or a TMA store will read, before the hand-off arrival;
//  * after ld.shared from a TMA-written stage, before the arrival that lets TMA refill it.  An mbarrier
//    arrival alone does not order the refill behind those loads; under memory-system pressure the
//    refill has been seen to land first, and the loads returned the next tile's data.
// Stages that only the async proxy reads (TMA -> tcgen05.mma) need no fence; tcgen05.commit orders them.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA (tiled mode; every block issues its own loads) -------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_load_5d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1,
                                            int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], "
        "[%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// Tensor store shared -> global (bulk async group).  Out-of-range parts of the box are
// clipped.  The issuing thread must commit the group and, before the shared buffer is
// overwritten, wait until the group has finished reading it.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, const void *smem_src, int c0, int c1, int c2,
                                             int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until at most `Pending` of this thread's committed store groups still read shared memory.
template <int Pending>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Pending) : "memory");
}

template <int Pending>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(Pending) : "memory");
}

// Barrier among a subset of the block's warps (id 1..15, thread count a multiple of 32).
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- tensor memory ------------------------------------------------------------
// Whole-warp calls (.sync.aligned).  `columns` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane
// (taddr.lane + t), columns taddr.col .. taddr.col + 31.  A warp may only
// address the lane quarter 32 * (warp_id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Registers -> tensor memory, same shape as tmem_ld_32x32.  The stores are complete (visible
// to a later tcgen05.mma after the usual fence / barrier hand-off) once tmem_st_wait returns.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- tcgen05.mma --------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle.  `addr` is the shared
// address of the first byte the instruction should read; lbo/sbo are the
// leading / stride byte offsets of the canonical layout:
//   K-major  : rows of 128 B (32 f32 along K), 8 rows per 1024 B atom;
//              sbo = distance between 8-row groups, lbo unused (1).
//   MN-major : rows of 128 B (32 f32 along M or N), 8 K-rows per 1024 B atom;
//              lbo = distance between 32-element groups along M/N,
//              sbo = distance between 8-row groups along K.
//
// 32-bit operands that are MN-major must use the "128-byte swizzle with 32-byte
// atoms" variant instead (layout type 1, TMA swizzle 128B_ATOM_32B): 32-byte
// chunks of a 128 B row are XOR-ed with the row index mod 4, 4 K-rows form a
// 512 B atom, sbo = distance between 4-row groups along K.
constexpr uint32_t kLayoutSw128 = 2;
constexpr uint32_t kLayoutSw128Base32 = 1;

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;  // descriptor version of sm_100
    d |= static_cast<uint64_t>(layout_type) << 61;
    return d;
}

__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return smem_desc(addr, lbo_bytes, sbo_bytes, kLayoutSw128);
}

// Instruction descriptor for kind::tf32 with an f32 accumulator.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4)                              // D format: f32
           | (2u << 7) | (2u << 10)               // A and B format: tf32
           | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16)
           | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues it for the whole CTA.
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         bool accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
}

// Same with the A operand in tensor memory (lane = row, one 32-bit column per K element;
// A is always K-major in this form).
__device__ __forceinline__ void mma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            bool accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

}  // namespace sm100

// ---- host side: tensor maps ----------------------------------------------------
// cuTensorMapEncodeTiled is fetched through the runtime so the library does not
// link against libcuda directly.
typedef CUresult (*katsu_tensor_map_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                               const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                               const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline katsu_tensor_map_encode_fn katsu_tensor_map_encoder() {
    static katsu_tensor_map_encode_fn fn = nullptr;
    if (fn == nullptr) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<katsu_tensor_map_encode_fn>(sym);
    }
    return fn;
}

// f32 tensor of `rank` dimensions (dims[0] innermost, strides in elements for
// dims 1..rank-1), box extents in elements, 128-byte swizzle, zero fill outside.
static inline bool katsu_make_tensor_map(CUtensorMap *map, const float *base, int rank, const uint64_t *dims,
                                         const uint64_t *strides_elems, const uint32_t *box,
                                         CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    if (rank < 1 || rank > 5) return false;
    katsu_tensor_map_encode_fn encode = katsu_tensor_map_encoder();
    if (encode == nullptr) return false;
    cuuint64_t gdims[5], gstrides[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstrides[i - 1] = strides_elems[i] * sizeof(float);
    }
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<float *>(base), gdims, gstrides,
                  gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
