// QVB8 prefill for sm_100a: Y (M, Q) fp32 = X (M, P) @ W^T for hundreds to thousands of tokens, the weight tile restored
// from the packed ids inside the kernel and contracted on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory).
//
// Replaces the reference's M > 8 path (formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:1542-1671: restore the whole
// weight to fp16 in HBM, then cublasGemmEx fp16 x fp16 -> fp32).  Arithmetic here: the factored form the small-M
// kernels use, y[m, q] = tau_s[q] * sum_c x[m, c] * id[q, c] + min_s[q] * sum_c x[m, c]: the ids are exact in fp16, X is
// narrowed to saturated fp16 first (:761-841), products are exact and accumulated in fp32, so the weight enters
// un-narrowed (the reference rounds it once to fp16; both are within the certificate).  Rows wider than 11 bits, whose
// ids fp16 cannot hold exactly, are recomputed in fp32 afterwards; escapes are then added from the plan's differences
// (exact - band), one thread per (row, token) in stored order.
//
// Tiling: a CTA owns 128 consecutive output rows and up to 256 tokens; K advances in blocks of 64 columns through two
// shared-memory stages.  Per block all 256 threads unpack the 128 x 64 ids (a thread produces one 16-byte row of an
// 8 x 16-byte core matrix: 8 ids = nb whole bytes of the row) and copy the 256 x 64 activations into the K-major
// no-swizzle canonical layout; one thread then issues four tcgen05.mma (128 x 256 x 16) and commits them to the
// stage's mbarrier, which frees the stage.  The 128 x 256 fp32 accumulator lives in 256 columns of tensor memory; at
// the end four warps read it with tcgen05.ld (a warp owns 32 lanes = 32 output rows) and write Y.
//
// Waits are bounded: a wait that runs out raises an abort flag and the error word, everybody falls through, and the
// tensor memory is released before the CTA exits.
#include "common.cuh"

namespace qv {

constexpr int PF_ROWS = 128;               // output rows per CTA = MMA M
constexpr int PF_TOK = 256;                // tokens per CTA = MMA N = tensor-memory columns
constexpr int PF_BK = 64;                  // columns per stage
constexpr int PF_THREADS = 256;
constexpr int PF_A_BYTES = PF_ROWS * PF_BK * 2;     // 16 KB
constexpr int PF_B_BYTES = PF_TOK * PF_BK * 2;      // 32 KB
constexpr int PF_STAGE = PF_A_BYTES + PF_B_BYTES;
constexpr int PF_SPIN = 1 << 22;

__device__ int g_prefill_error = 0;

void plan_escape_sections(const void *plan, int64_t Q, int64_t n_esc, const int **esc_ptr, const int **esc_col,
                          const float **esc_delta);                 // qvb8_small_m.cu

__device__ __forceinline__ uint32_t pf_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool pf_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    return ok != 0;
}
__device__ __noinline__ bool pf_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    uint64_t t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (int i = 0; i < PF_SPIN; ++i) {
        if (pf_try_wait(bar, parity)) return true;
        if ((i & 7) == 7) {
            if (*abort_flag) return false;
            uint64_t t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            if (t - t0 > 2000000000ull) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_prefill_error, 0, code);
    return false;
}

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes stored as 128 contiguous
// bytes; `sbo` bytes between core matrices along the rows, `lbo` bytes between core matrices along K; version 1.
__device__ __forceinline__ uint64_t pf_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

struct PrefillParams {
    const uint8_t *ids;
    const float *min_s, *tau_s;
    const uint8_t *nbits;
    const int64_t *bit_off;
    const __half *X16;         // (M, P) saturated fp16
    const float *sumx;         // (M) sums of the narrowed activations
    float *Y;                  // (M, Q)
    int Q, P, M;
};

__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ alignas(8) uint64_t mma_done[2];        // the MMAs that read stage s have completed
    __shared__ alignas(8) uint64_t all_done;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_word;
    volatile int *abort_flag = &abort_word;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q0 = blockIdx.x * PF_ROWS, n0 = blockIdx.y * PF_TOK;
    if (tid == 0) {
        for (int s = 0; s < 2; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&mma_done[s])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&all_done)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_word = 0;
    }
    if (warp == 0) {                                    // one warp allocates (and later frees) the tensor-memory columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(pf_smem(&tmem_base)), "r"((uint32_t)PF_TOK) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base;

    // instruction descriptor: fp32 accumulate, fp16 x fp16, both operands K-major, N = 256, M = 128
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(PF_TOK >> 3) << 17) | ((uint32_t)(PF_ROWS >> 4) << 24);

    // this thread's weight row (fixed for the whole kernel): row r of the tile, K-groups j0, j0 + 2, j0 + 4, j0 + 6
    const int r = tid & 127, j0 = tid >> 7;
    const int q = q0 + r;
    const bool row_ok = q < p.Q;
    const int nb = row_ok ? __ldg(p.nbits + q) : 1;
    const int64_t bit0 = row_ok ? __ldg(p.bit_off + q) : 0;
    const bool fast = nb <= 8 && (bit0 & 7) == 0;
    const uint32_t mask = (1u << nb) - 1u;
    // this thread's token (fixed): token n of the tile, all 8 K-groups
    const int n = n0 + tid;
    const bool tok_ok = n < p.M;
    const __half *xrow = p.X16 + (int64_t)(tok_ok ? n : 0) * p.P;

    const int nkb = p.P / PF_BK;
    bool alive = true;
    for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb & 1;
        uint8_t *A = smem + s * PF_STAGE, *B = A + PF_A_BYTES;
        // the MMAs issued two blocks ago read this stage: wait until they are done
        if (kb >= 2 && alive) alive = pf_wait(pf_smem(&mma_done[s]), ((kb >> 1) - 1) & 1, abort_flag, 21);
        const int k0 = kb * PF_BK;
        // ---- weights: ids as fp16 integers, layout [K-group][row] x 16 bytes
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int j = j0 + 2 * it;
            uint32_t h[4] = {0u, 0u, 0u, 0u};
            if (row_ok) {
                const int col = k0 + 8 * j;
                if (fast) {
                    const int64_t a = (bit0 >> 3) + (int64_t)(col >> 3) * nb;
                    const uint64_t *w = reinterpret_cast<const uint64_t *>(p.ids + (a & ~(int64_t)7));
                    const uint64_t lo = __ldg(w), hi = __ldg(w + 1);
                    const int sh = (int)(a & 7) * 8;
                    const uint64_t v = sh ? (lo >> sh) | (hi << (64 - sh)) : lo;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t a0 = (uint32_t)(v >> ((2 * i) * nb)) & mask, a1 = (uint32_t)(v >> ((2 * i + 1) * nb)) & mask;
                        const __half2 hh = __halves2half2(__ushort2half_rn((unsigned short)a0), __ushort2half_rn((unsigned short)a1));
                        h[i] = *reinterpret_cast<const uint32_t *>(&hh);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t a0 = field_bytes(p.ids, bit0 + (int64_t)(col + 2 * i) * nb, nb);
                        const uint32_t a1 = field_bytes(p.ids, bit0 + (int64_t)(col + 2 * i + 1) * nb, nb);
                        const __half2 hh = __halves2half2(__ushort2half_rn((unsigned short)a0), __ushort2half_rn((unsigned short)a1));
                        h[i] = *reinterpret_cast<const uint32_t *>(&hh);
                    }
                }
            }
            *reinterpret_cast<uint4 *>(A + j * (PF_ROWS * 16) + r * 16) = make_uint4(h[0], h[1], h[2], h[3]);
        }
        // ---- activations: layout [K-group][token] x 16 bytes
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (tok_ok) v = __ldg(reinterpret_cast<const uint4 *>(xrow + k0 + 8 * j));
            *reinterpret_cast<uint4 *>(B + j * (PF_TOK * 16) + tid * 16) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // generic-proxy writes -> visible to the MMA
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
        if (tid == 0 && alive) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t a32 = pf_smem(A), b32 = pf_smem(B);
#pragma unroll
            for (int kk = 0; kk < PF_BK / 16; ++kk) {
                // one MMA covers two K-groups: core matrices 2 kk and 2 kk + 1
                const uint64_t da = pf_desc(a32 + 2 * kk * (PF_ROWS * 16), PF_ROWS * 16, 128);
                const uint64_t db = pf_desc(b32 + 2 * kk * (PF_TOK * 16), PF_TOK * 16, 128);
                const uint32_t accumulate = (kb > 0 || kk > 0) ? 1u : 0u;
                asm volatile(
                    "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                    " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n"
                    :: "r"(tmem), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(pf_smem(&mma_done[s])) : "memory");
            if (kb == nkb - 1)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(pf_smem(&all_done)) : "memory");
        }
    }
    // ---- epilogue: tensor memory -> registers -> Y
    if (alive) alive = pf_wait(pf_smem(&all_done), 0, abort_flag, 22);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (warp < 4 && alive) {
        const int qr = q0 + warp * 32 + lane;               // tensor-memory lane = row of the tile
        const bool ok = qr < p.Q;
        const float ts = ok ? __ldg(p.tau_s + qr) : 0.f, ms = ok ? __ldg(p.min_s + qr) : 0.f;
        for (int c0 = 0; c0 < PF_TOK; c0 += 32) {
            uint32_t d[32];
            const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
                  "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]), "=r"(d[16]),
                  "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]), "=r"(d[24]),
                  "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int nn = n0 + c0 + j;
                if (ok && nn < p.M) p.Y[(int64_t)nn * p.Q + qr] = __fmaf_rn(ts, __uint_as_float(d[j]), ms * __ldg(p.sumx + nn));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"((uint32_t)PF_TOK) : "memory");
}

// X (M, P) of any input type -> saturated fp16 copy and the per-token sums of the narrowed values (fixed order: one
// warp per token, lane-strided, then a shuffle tree)
__global__ void __launch_bounds__(256) prefill_narrow_kernel(const void *__restrict__ X, int x_dtype, int M, int P,
                                                             __half *__restrict__ X16, float *__restrict__ sumx) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    float s = 0.f;
    for (int c = lane; c < P; c += 32) {
        const int64_t i = (int64_t)warp * P + c;
        const float v = x_dtype == QVB8_F32 ? __ldg(reinterpret_cast<const float *>(X) + i)
                      : x_dtype == QVB8_BF16 ? __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16 *>(X) + i))
                                             : __half2float(__ldg(reinterpret_cast<const __half *>(X) + i));
        const __half h = sat_half(v);
        X16[i] = h;
        s += __half2float(h);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) sumx[warp] = s;
}

// Y[m, q] += sum over the escapes of row q of x16[m, col] * (exact - band), in stored order
__global__ void __launch_bounds__(256) prefill_escapes_kernel(const int *__restrict__ esc_ptr, const int *__restrict__ esc_col,
                                                              const float *__restrict__ esc_delta, const __half *__restrict__ X16,
                                                              float *__restrict__ Y, int Q, int P, int M) {
    const int q = blockIdx.x;
    const int e0 = __ldg(esc_ptr + q), e1 = __ldg(esc_ptr + q + 1);
    if (e0 == e1) return;
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        float a = 0.f;
        for (int e = e0; e < e1; ++e) a = __fmaf_rn(__half2float(X16[(int64_t)m * P + __ldg(esc_col + e)]), __ldg(esc_delta + e), a);
        Y[(int64_t)m * Q + q] += a;
    }
}

// Rows wider than 11 bits: their ids are not exact in fp16 (integers above 2048 are not all representable), so the
// tensor-core result of such a row is replaced by an fp32 product over the row.  They are rare (rows dominated by
// outliers).  First a compact list of them, then one warp per (wide row, token).
constexpr int PF_EXACT_BITS = 11;
__global__ void __launch_bounds__(256) prefill_wide_list_kernel(const uint8_t *__restrict__ nbits, int Q, int *__restrict__ list,
                                                                int *__restrict__ count) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q < Q && __ldg(nbits + q) > PF_EXACT_BITS) list[atomicAdd(count, 1)] = q;
}
__global__ void __launch_bounds__(256) prefill_wide_rows_kernel(const PrefillParams p, const int *__restrict__ list,
                                                                const int *__restrict__ count) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.y * 8 + warp;
    if (m >= p.M) return;
    const int n = *count;
    for (int wi = blockIdx.x; wi < n; wi += gridDim.x) {
        const int q = list[wi];
        const int nb = __ldg(p.nbits + q);
        const int64_t bit0 = __ldg(p.bit_off + q);
        const float ts = __ldg(p.tau_s + q), ms = __ldg(p.min_s + q);
        float a = 0.f;
        for (int c = lane; c < p.P; c += 32)
            a = __fmaf_rn(__half2float(p.X16[(int64_t)m * p.P + c]), band(field_bytes(p.ids, bit0 + (int64_t)c * nb, nb), ts, ms), a);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0) p.Y[(int64_t)m * p.Q + q] = a;
    }
}

int prefill_error_word(int *out) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_prefill_error, sizeof(int)) != cudaSuccess) return cuda_status("qvb8_device_status");
    *out = v;
    return QVB8_OK;
}

}  // namespace qv

QV_API int64_t qvb8_prefill_scratch_bytes(int64_t M, int64_t Q, int64_t P) {
    if (M <= 0 || P <= 0 || Q < 0) return 0;
    return (M * P * 2 + 255) / 256 * 256 + (M * 4 + 255) / 256 * 256 + ((Q + 1) * 4 + 255) / 256 * 256;
}

QV_API int qvb8_prefill(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int64_t M, float *Y, void *scratch,
                        int64_t scratch_bytes, void *stream) {
    using namespace qv;
    if (int rc = check_pack(w, "qvb8_prefill")) return rc;
    if (int rc = check_device("qvb8_prefill")) return rc;
    if (!X || !Y || M <= 0 || M > 0x7fffffff) return fail(QVB8_ERR_ARG, "qvb8_prefill: bad X / Y / M");
    if (x_dtype != QVB8_F16 && x_dtype != QVB8_BF16 && x_dtype != QVB8_F32) return fail(QVB8_ERR_ARG, "qvb8_prefill: bad X dtype");
    if (w->Q == 0) return QVB8_OK;
    if (w->P % PF_BK != 0) return fail(QVB8_ERR_ARG, "qvb8_prefill: P must be a multiple of %d", PF_BK);
    if (w->n_esc > 0 && !plan) return fail(QVB8_ERR_ARG, "qvb8_prefill: a pack with escapes needs its plan (qvb8_plan_build)");
    const int64_t need = qvb8_prefill_scratch_bytes(M, w->Q, w->P);
    if (!scratch || scratch_bytes < need || !aligned(scratch, 256))
        return fail(QVB8_ERR_SCRATCH, "qvb8_prefill: scratch of %lld bytes (256-byte aligned) needed, %lld given", (long long)need, (long long)scratch_bytes);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    __half *X16 = reinterpret_cast<__half *>(scratch);
    float *sumx = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scratch) + (M * w->P * 2 + 255) / 256 * 256);
    int *wide = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(sumx) + (M * 4 + 255) / 256 * 256);      // [0] count, then rows
    prefill_narrow_kernel<<<(unsigned)((M * 32 + 255) / 256), 256, 0, st>>>(X, x_dtype, (int)M, (int)w->P, X16, sumx);
    if (int rc = cuda_status("qvb8_prefill narrow")) return rc;
    static thread_local int granted_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != granted_dev) {
        if (cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * PF_STAGE + 1024) != cudaSuccess)
            return cuda_status("qvb8_prefill: shared memory opt-in");
        granted_dev = dev;
    }
    PrefillParams prm{w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, X16, sumx, Y, (int)w->Q, (int)w->P, (int)M};
    const dim3 grid((unsigned)((w->Q + PF_ROWS - 1) / PF_ROWS), (unsigned)((M + PF_TOK - 1) / PF_TOK));
    prefill_kernel<<<grid, PF_THREADS, 2 * PF_STAGE + 1024, st>>>(prm);
    if (int rc = cuda_status("qvb8_prefill")) return rc;
    if (cudaMemsetAsync(wide, 0, sizeof(int), st) != cudaSuccess) return cuda_status("qvb8_prefill memset");
    prefill_wide_list_kernel<<<(unsigned)((w->Q + 255) / 256), 256, 0, st>>>(w->nbits, (int)w->Q, wide + 1, wide);
    prefill_wide_rows_kernel<<<dim3(64, (unsigned)((M + 7) / 8)), 256, 0, st>>>(prm, wide + 1, wide);
    if (int rc = cuda_status("qvb8_prefill wide rows")) return rc;
    if (w->n_esc > 0) {
        const int *esc_ptr, *esc_col;
        const float *esc_delta;
        plan_escape_sections(plan, w->Q, w->n_esc, &esc_ptr, &esc_col, &esc_delta);
        prefill_escapes_kernel<<<(unsigned)w->Q, 256, 0, st>>>(esc_ptr, esc_col, esc_delta, X16, Y, (int)w->Q, (int)w->P, (int)M);
        if (int rc = cuda_status("qvb8_prefill escapes")) return rc;
    }
    return QVB8_OK;
}
