// One-shot all-reduce of the small partial results of the row-parallel projections (o, down) over NVLink peer memory.
//
// The reference splits a linear across cards by output rows and exchanges with NCCL at the shard boundary
// (formats/qvb8/module.py:126-160 row_subset, run/placement.py).  For decode the exchanged vector is tiny (M x d_model
// fp32 = 16 .. 256 KB), so the cost of a library all-reduce is its latency.  Here every rank PUSHES its partial sums
// straight into a receive slot on every peer (plain peer stores, no multicast), raises a flag there, waits for the
// peers' flags, and adds the slots up in rank order: every rank gets bit-identical sums.
//
// Memory of a rank (one allocation, shared with the peers through CUDA IPC):
//   [0, 8192)                       flags[2][world][32 blocks]: flag[b][r][k] = last epoch whose slice k rank r has put
//                                   into buffer b; one word at the end counts this rank's finished blocks
//   [8192 + b * world * cap ...)    recv[b][r][cap floats]: the partial sums of rank r for an epoch of parity b
// A call is cut into up to 32 blocks; block k exchanges slice k of the vector with the peers' blocks k and depends on
// no other block of its own grid (so the blocks need not be resident together).
// Two buffers: a rank can run at most one all-reduce ahead of a peer (it needs the peer's flag of the current epoch,
// which the peer raises only after it has finished reading the previous one).
//
// Waits are bounded (2 s): a wait that runs out raises the error word and the kernel carries on with what it has.
#include "common.cuh"

#include <cstring>

namespace qv {

constexpr int PEER_MAX_WORLD = 16;
constexpr int PEER_FLAG_BYTES = 8192;          // flags[2][world][PEER_MAX_BLOCKS] + the blocks-done counter
constexpr int PEER_MAX_BLOCKS = 32;           // blocks one all-reduce is cut into (each exchanges its own slice)
constexpr int PEER_THREADS = 1024;

__device__ int g_peer_error = 0;

struct PeerParams {
    uint8_t *base[PEER_MAX_WORLD];       // every rank's allocation as mapped in THIS process (base[rank] = own)
    int rank, world;
    int64_t cap;                         // floats per receive slot
    uint32_t *epoch;                     // device counter of this rank: all-reduces done so far
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

// Block k of `nblk` handles floats [k * per, min(n, (k + 1) * per)), per a multiple of 4.  n a multiple of 4, n <= cap.
// `partial` and `out` may be the same buffer (every thread reads the elements it later writes), so neither is declared
// restrict.  wait_ns: how long the wait for the peers' flags may last before it gives up (error word 31); the time
// limit is what bounds the wait, the iteration cap only guards against a timer that does not advance.
__device__ __forceinline__ void peer_allreduce_body(const PeerParams &p, int rank, uint32_t *epoch_ctr, const float *partial,
                                                    float *out, int n, uint64_t wait_ns, int k, int nblk,
                                                    bool gather = false) {
    __shared__ uint32_t s_epoch;
    const int tid = threadIdx.x;
    if (tid == 0) s_epoch = *epoch_ctr + 1u;              // (advanced only after every block of this call has read it)
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int b = (int)(epoch & 1u);
    const int per = ((n / 4 + nblk - 1) / nblk) * 4;
    const int lo = min(n, k * per), hi = min(n, lo + per);
    const int64_t slot = ((int64_t)b * p.world + rank) * p.cap;
    // 1. push: this rank's slice into slot [b][rank] of every rank (its own included)
    const float4 *src = reinterpret_cast<const float4 *>(partial);
    for (int j = 0; j < p.world; ++j) {
        const int r = (rank + j) % p.world;               // every rank starts with another peer
        float4 *dst = reinterpret_cast<float4 *>(p.base[r] + PEER_FLAG_BYTES) + (slot >> 2);
        for (int i = (lo >> 2) + tid; i < (hi >> 2); i += PEER_THREADS) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    // 2. flags: tell every rank that this rank's slice of this epoch is in place
    const int fidx = (b * PEER_MAX_WORLD + rank) * PEER_MAX_BLOCKS + k;
    if (tid < p.world) st_release_sys(reinterpret_cast<uint32_t *>(p.base[tid]) + fidx, epoch);
    // 3. wait for every rank's flag of this slice in this rank's memory
    if (tid < p.world) {
        const uint32_t *f = reinterpret_cast<const uint32_t *>(p.base[rank]) + (b * PEER_MAX_WORLD + tid) * PEER_MAX_BLOCKS + k;
        uint64_t t0, t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        bool ok = false;
        for (long long i = 0; i < (1ll << 34); ++i) {
            if ((int32_t)(ld_acquire_sys(f) - epoch) >= 0) { ok = true; break; }
            if ((i & 15) == 15) {
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
                if (t - t0 > wait_ns) break;
            }
        }
        if (!ok) atomicCAS(&g_peer_error, 0, 31);
    }
    __syncthreads();
    // 4. sum the slots in rank order (all-gather: lay them side by side, rank r's n floats at out[r * n])
    const float4 *rb = reinterpret_cast<const float4 *>(p.base[rank] + PEER_FLAG_BYTES) + (((int64_t)b * p.world * p.cap) >> 2);
    if (gather) {
        for (int r = 0; r < p.world; ++r) {
            const float4 *from = rb + (((int64_t)r * p.cap) >> 2);
            float4 *to = reinterpret_cast<float4 *>(out) + (((int64_t)r * n) >> 2);
            for (int i = (lo >> 2) + tid; i < (hi >> 2); i += PEER_THREADS) to[i] = from[i];
        }
    } else
    for (int i = (lo >> 2) + tid; i < (hi >> 2); i += PEER_THREADS) {
        float4 a = rb[i];
        for (int r = 1; r < p.world; ++r) {
            const float4 v = rb[(((int64_t)r * p.cap) >> 2) + i];
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        reinterpret_cast<float4 *>(out)[i] = a;
    }
    // 5. the block that finishes last advances the epoch (every block has read it by then)
    __syncthreads();
    if (tid == 0) {
        uint32_t *done = reinterpret_cast<uint32_t *>(p.base[rank] + PEER_FLAG_BYTES - 4);   // (the flags end at byte 4096)
        __threadfence();
        if (atomicAdd(done, 1u) == (uint32_t)nblk - 1u) {
            *done = 0u;
            __threadfence();
            *epoch_ctr = epoch;
        }
    }
}

__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_kernel(const PeerParams p, const float *partial, float *out,
                                                                      int n, uint64_t wait_ns, int gather) {
    // programmatic dependent launch: the next kernel may begin its prologue now (it waits for this grid's completion
    // before it reads anything this grid writes); this grid waits for its predecessor before it reads `partial`
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    peer_allreduce_body(p, p.rank, p.epoch, partial, out, n, wait_ns, blockIdx.x, gridDim.x, gather != 0);
}

// All ranks of a world in ONE cooperative launch on one device, block r = rank r: the protocol exactly as above, for
// machines with fewer GPUs than ranks (blocks of a cooperative launch are co-resident, so their waits on one another
// end; separate launches that wait on one another carry no such guarantee).
struct PeerLocalRanks {
    const float *partial[PEER_MAX_WORLD];
    float *out[PEER_MAX_WORLD];
    uint32_t *epoch[PEER_MAX_WORLD];
};
__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_local_kernel(const PeerParams p, const PeerLocalRanks l, int n,
                                                                            uint64_t wait_ns, int gather) {
    const int rank = blockIdx.x;
    peer_allreduce_body(p, rank, l.epoch[rank], l.partial[rank], l.out[rank], n, wait_ns, 0, 1, gather != 0);
}

int peer_error_word(int *out) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_error, sizeof(int)) != cudaSuccess) return cuda_status("qvb8_device_status");
    *out = v;
    return QVB8_OK;
}

int peer_error_reset() {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_peer_error, &zero, sizeof(int)) != cudaSuccess) return cuda_status("qvb8_device_status_reset");
    return QVB8_OK;
}

}  // namespace qv

QV_API int64_t qvb8_peer_bytes(int world, int64_t cap_floats) {
    if (world < 1 || world > qv::PEER_MAX_WORLD || cap_floats < 4) return 0;
    cap_floats = (cap_floats + 3) / 4 * 4;
    return qv::PEER_FLAG_BYTES + 2 * (int64_t)world * cap_floats * 4 + 256;
}

/* Allocates (cudaMalloc, zeroed) this rank's exchange memory on the current device and returns its IPC handle (64
 * bytes) for the peers. */
QV_API int qvb8_peer_alloc(int64_t bytes, void **ptr, unsigned char handle[64]) {
    using namespace qv;
    if (int rc = check_device("qvb8_peer_alloc")) return rc;
    if (!ptr || !handle || bytes <= 0) return fail(QVB8_ERR_ARG, "qvb8_peer_alloc: bad arguments");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    static_assert(2 * PEER_MAX_WORLD * PEER_MAX_BLOCKS * 4 <= PEER_FLAG_BYTES - 4, "flag area");
    if (cudaMalloc(ptr, (size_t)bytes) != cudaSuccess) return cuda_status("qvb8_peer_alloc");
    if (cudaMemset(*ptr, 0, (size_t)bytes) != cudaSuccess) return cuda_status("qvb8_peer_alloc memset");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) return cuda_status("qvb8_peer_alloc handle");
    memcpy(handle, &h, 64);
    return cudaDeviceSynchronize() == cudaSuccess ? QVB8_OK : cuda_status("qvb8_peer_alloc sync");
}

QV_API int qvb8_peer_open(const unsigned char handle[64], void **ptr) {
    using namespace qv;
    if (int rc = check_device("qvb8_peer_open")) return rc;
    if (!ptr || !handle) return fail(QVB8_ERR_ARG, "qvb8_peer_open: bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return cuda_status("qvb8_peer_open");
    return QVB8_OK;
}

QV_API int qvb8_peer_close(void *ptr, int own) {
    if (!ptr) return QVB8_OK;
    const cudaError_t e = own ? cudaFree(ptr) : cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? QVB8_OK : qv::cuda_status("qvb8_peer_close");
}

/* out[0 .. n) = sum over the ranks of their partial[0 .. n), identical on every rank.  bases[r] = rank r's exchange
 * memory as mapped in this process (own allocation for r = rank); epoch = a zeroed uint32 of this rank in device
 * memory, owned by the communicator.  n % 4 == 0, n <= cap_floats.  Every rank must make the same sequence of calls.
 * flags: QVB8_FLAG_PDL launches with programmatic stream serialization, like qvb8_small_m_ex.
 * wait_ns: how long the kernel waits for the peers' flags before it gives up with error word 31 (0 = two seconds). */
namespace qv {
constexpr uint64_t PEER_WAIT_NS = 2000000000ull;
static int peer_fill(PeerParams &p, void *const *bases, int rank, int world, int64_t &cap_floats, int64_t n, const char *who) {
    if (!bases || world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world)
        return fail(QVB8_ERR_ARG, "%s: bad arguments", who);
    cap_floats = (cap_floats + 3) / 4 * 4;
    if (n <= 0 || n % 4 != 0 || n > cap_floats) return fail(QVB8_ERR_ARG, "%s: n must be a multiple of 4 within the slot size", who);
    for (int r = 0; r < world; ++r) {
        if (!bases[r]) return fail(QVB8_ERR_ARG, "%s: null peer mapping", who);
        p.base[r] = reinterpret_cast<uint8_t *>(bases[r]);
    }
    p.rank = rank;
    p.world = world;
    p.cap = cap_floats;
    return QVB8_OK;
}
}  // namespace qv

namespace qv {
static int peer_exchange(void *const *bases, int rank, int world, int64_t cap_floats, void *epoch, const float *partial,
                         float *out, int64_t n, int flags, uint64_t wait_ns, void *stream, int gather) {
    if (int rc = check_device("qvb8_peer_allreduce")) return rc;
    if (!epoch || !partial || !out) return fail(QVB8_ERR_ARG, "qvb8_peer_allreduce: bad arguments");
    PeerParams p{};
    if (int rc = peer_fill(p, bases, rank, world, cap_floats, n, "qvb8_peer_allreduce")) return rc;
    if (!aligned(partial, 16) || !aligned(out, 16)) return fail(QVB8_ERR_ARG, "qvb8_peer_allreduce: partial / out must be 16-byte aligned");
    p.epoch = reinterpret_cast<uint32_t *>(epoch);
    cudaLaunchConfig_t cfg{};
    // one block per 4 K floats (one 16-byte store per thread and peer), at most PEER_MAX_BLOCKS: a decode-sized vector
    // stays one block, the partial sums of several layers exchanged at once spread over many SMs (one SM's stores
    // would otherwise bound the push)
    int nblk = (int)((n + 4095) / 4096);
    if (nblk > PEER_MAX_BLOCKS) nblk = PEER_MAX_BLOCKS;
    cfg.gridDim = dim3(nblk);
    cfg.blockDim = dim3(PEER_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & QVB8_FLAG_PDL) ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, p, partial, out, (int)n, wait_ns ? wait_ns : PEER_WAIT_NS, gather) !=
        cudaSuccess)
        return cuda_status("qvb8_peer_allreduce launch");
    return cuda_status("qvb8_peer_allreduce");
}
}  // namespace qv

QV_API int qvb8_peer_allreduce_ex(void *const *bases, int rank, int world, int64_t cap_floats, void *epoch,
                                  const float *partial, float *out, int64_t n, int flags, uint64_t wait_ns, void *stream) {
    return qv::peer_exchange(bases, rank, world, cap_floats, epoch, partial, out, n, flags, wait_ns, stream, 0);
}

/* All-gather with the same protocol: out[r * n .. (r + 1) * n) = rank r's part[0 .. n), identical on every rank.  `out`
 * holds world * n floats and must not overlap `part`.  The two kinds of exchange may be mixed on one communicator (they
 * share the epoch counter); every rank must make the same sequence of calls. */
QV_API int qvb8_peer_allgather(void *const *bases, int rank, int world, int64_t cap_floats, void *epoch, const float *part,
                               float *out, int64_t n, int flags, uint64_t wait_ns, void *stream) {
    return qv::peer_exchange(bases, rank, world, cap_floats, epoch, part, out, n, flags, wait_ns, stream, 1);
}

QV_API int qvb8_peer_allreduce(void *const *bases, int rank, int world, int64_t cap_floats, void *epoch, const float *partial,
                               float *out, int64_t n, int flags, void *stream) {
    return qvb8_peer_allreduce_ex(bases, rank, world, cap_floats, epoch, partial, out, n, flags, 0, stream);
}

/* Every rank of a `world` on ONE device in one cooperative launch (block r acts as rank r): bases[r], epochs[r],
 * partials[r], outs[r] are rank r's exchange area, epoch counter, input and output, all in this device's memory.  For
 * machines with fewer GPUs than ranks: kernels that wait on one another must not run as separate launches on one
 * GPU, the blocks of a cooperative launch may. */
namespace qv {
static int peer_exchange_local(void *const *bases, int world, int64_t cap_floats, void *const *epochs,
                               const float *const *partials, float *const *outs, int64_t n, uint64_t wait_ns, void *stream,
                               int gather) {
    if (int rc = check_device("qvb8_peer_allreduce_local")) return rc;
    if (!epochs || !partials || !outs) return fail(QVB8_ERR_ARG, "qvb8_peer_allreduce_local: bad arguments");
    PeerParams p{};
    if (int rc = peer_fill(p, bases, 0, world, cap_floats, n, "qvb8_peer_allreduce_local")) return rc;
    PeerLocalRanks l{};
    for (int r = 0; r < world; ++r) {
        if (!epochs[r] || !partials[r] || !outs[r] || !aligned(partials[r], 16) || !aligned(outs[r], 16))
            return fail(QVB8_ERR_ARG, "qvb8_peer_allreduce_local: null or unaligned buffer of rank %d", r);
        l.partial[r] = partials[r];
        l.out[r] = outs[r];
        l.epoch[r] = reinterpret_cast<uint32_t *>(epochs[r]);
    }
    int dev = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop) return fail(QVB8_ERR_ARG, "qvb8_peer_allreduce_local: the device has no cooperative launch");
    int nn = (int)n;
    uint64_t wn = wait_ns ? wait_ns : PEER_WAIT_NS;
    void *args[] = {&p, &l, &nn, &wn, &gather};
    if (cudaLaunchCooperativeKernel((const void *)peer_allreduce_local_kernel, dim3(world), dim3(PEER_THREADS), args, 0,
                                    reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess)
        return cuda_status("qvb8_peer_allreduce_local launch");
    return cuda_status("qvb8_peer_allreduce_local");
}
}  // namespace qv

QV_API int qvb8_peer_allreduce_local(void *const *bases, int world, int64_t cap_floats, void *const *epochs,
                                     const float *const *partials, float *const *outs, int64_t n, uint64_t wait_ns,
                                     void *stream) {
    return qv::peer_exchange_local(bases, world, cap_floats, epochs, partials, outs, n, wait_ns, stream, 0);
}

/* The all-gather of every rank of a `world` on one device, as qvb8_peer_allreduce_local does for the all-reduce. */
QV_API int qvb8_peer_allgather_local(void *const *bases, int world, int64_t cap_floats, void *const *epochs,
                                     const float *const *parts, float *const *outs, int64_t n, uint64_t wait_ns,
                                     void *stream) {
    return qv::peer_exchange_local(bases, world, cap_floats, epochs, parts, outs, n, wait_ns, stream, 1);
}
