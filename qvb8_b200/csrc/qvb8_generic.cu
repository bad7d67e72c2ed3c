// Layout-agnostic QVB8 small-M product and the escape correction shared by every small-M path.
//
//   Y[m, q] = sum_c X[m, c] * fma(id[q, c], tau_s[q], min_s[q])
//
// One warp per output row, one id per lane per step read byte-wise, so any P, any base alignment and any row
// width 1..14 work.  This is the fallback for packs the streaming kernel (qvb8_small_m.cu) cannot take; it is not
// tuned.  Follows the arithmetic of the reference GEMV (formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:418-452):
// fp32 band value, fp32 accumulation, activation narrowed to saturated fp16 first.
#include "common.cuh"

namespace qv {

constexpr int GEN_MB = 8;   // rows of X handled per pass

template <int XT>
__device__ __forceinline__ float x_value(const void *__restrict__ X, int64_t i, int x_mode) {
    const float v = load_x<XT>(X, i);
    return x_mode == 0 ? __half2float(sat_half(v)) : v;
}

template <int XT>
__global__ void __launch_bounds__(256) small_m_generic_kernel(const uint8_t *__restrict__ ids,
                                                              const float *__restrict__ min_s,
                                                              const float *__restrict__ tau_s,
                                                              const uint8_t *__restrict__ nbits,
                                                              const int64_t *__restrict__ bit_off,
                                                              const void *__restrict__ X, int x_mode, int m0, int mcount,
                                                              float *__restrict__ Y, int Q, int P) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t q = warp; q < Q; q += nwarps) {
        const int nb = __ldg(nbits + q);
        const int64_t base = __ldg(bit_off + q);
        const float m = __ldg(min_s + q), ts = __ldg(tau_s + q);
        float acc[GEN_MB];
#pragma unroll
        for (int r = 0; r < GEN_MB; ++r) acc[r] = 0.f;
        for (int c = lane; c < P; c += 32) {
            const float wv = band(field_bytes(ids, base + (int64_t)c * nb, nb), ts, m);
#pragma unroll
            for (int r = 0; r < GEN_MB; ++r)
                if (r < mcount) acc[r] = __fmaf_rn(x_value<XT>(X, (int64_t)(m0 + r) * P + c, x_mode), wv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < GEN_MB; ++r) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
            if (lane == 0 && r < mcount) Y[(int64_t)(m0 + r) * Q + q] = acc[r];
        }
    }
}

// Escapes: the banded pass multiplied the band value at positions whose exact value is stored separately.  Add
// x[m, c] * (exact - band) afterwards.  esc_idx is sorted, so the thread that holds the FIRST escape of an output
// row walks that row's run in order and writes each Y[m, q] once: no atomics, the same bits on every run.
// (The reference corrects the same way, qvb8_cuda.cu:507-533; here all M rows are handled by one launch.)
template <int XT>
__global__ void __launch_bounds__(128) fix_escapes_kernel(const uint8_t *__restrict__ ids, const float *__restrict__ min_s,
                                                          const float *__restrict__ tau_s,
                                                          const uint8_t *__restrict__ nbits,
                                                          const int64_t *__restrict__ bit_off,
                                                          const int64_t *__restrict__ esc_idx,
                                                          const float *__restrict__ esc_vals, int64_t n_esc,
                                                          const void *__restrict__ X, int x_mode, int M,
                                                          float *__restrict__ Y, int Q, int P) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_esc) return;
    const int64_t flat = __ldg(esc_idx + i);
    const int64_t q = flat / P;
    if (q < 0 || q >= Q) return;
    if (i > 0 && __ldg(esc_idx + i - 1) / P == q) return;
    const int nb = __ldg(nbits + q);
    const int64_t base = __ldg(bit_off + q);
    const float m = __ldg(min_s + q), ts = __ldg(tau_s + q);
    for (int m0 = 0; m0 < M; m0 += GEN_MB) {
        float a[GEN_MB];
#pragma unroll
        for (int r = 0; r < GEN_MB; ++r) a[r] = 0.f;
        for (int64_t e = i; e < n_esc; ++e) {
            const int64_t f = __ldg(esc_idx + e);
            if (f / P != q) break;
            const int c = (int)(f - q * P);
            const float d = __ldg(esc_vals + e) - band(field_bytes(ids, base + (int64_t)c * nb, nb), ts, m);
#pragma unroll
            for (int r = 0; r < GEN_MB; ++r)
                if (m0 + r < M) a[r] = __fmaf_rn(x_value<XT>(X, (int64_t)(m0 + r) * P + c, x_mode), d, a[r]);
        }
#pragma unroll
        for (int r = 0; r < GEN_MB; ++r)
            if (m0 + r < M) Y[(int64_t)(m0 + r) * Q + q] += a[r];
    }
}

int launch_fix_escapes(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y, cudaStream_t st) {
    if (w->n_esc <= 0) return QVB8_OK;
    const int grid = (int)((w->n_esc + 127) / 128);
#define QV_FIX(XT)                                                                                              \
    fix_escapes_kernel<XT><<<grid, 128, 0, st>>>(w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, w->esc_idx, \
                                                 w->esc_vals, w->n_esc, X, x_mode, M, Y, (int)w->Q, (int)w->P)
    if (x_dtype == QVB8_F16) QV_FIX(QVB8_F16);
    else if (x_dtype == QVB8_BF16) QV_FIX(QVB8_BF16);
    else QV_FIX(QVB8_F32);
#undef QV_FIX
    return cuda_status("qvb8 escape correction launch");
}

int launch_small_m_generic(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y,
                           cudaStream_t st) {
    const int Q = (int)w->Q, P = (int)w->P;
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = ((int64_t)Q + 7) / 8;
    const int grid = (int)(want < (int64_t)sms * 8 ? (want > 0 ? want : 1) : (int64_t)sms * 8);
    for (int m0 = 0; m0 < M; m0 += GEN_MB) {
        const int mc = M - m0 < GEN_MB ? M - m0 : GEN_MB;
#define QV_GEN(XT)                                                                                                 \
    small_m_generic_kernel<XT><<<grid, 256, 0, st>>>(w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, X, x_mode, \
                                                     m0, mc, Y, Q, P)
        if (x_dtype == QVB8_F16) QV_GEN(QVB8_F16);
        else if (x_dtype == QVB8_BF16) QV_GEN(QVB8_BF16);
        else QV_GEN(QVB8_F32);
#undef QV_GEN
        if (int rc = cuda_status("qvb8_small_m_generic launch")) return rc;
    }
    return launch_fix_escapes(w, X, x_dtype, x_mode, M, Y, st);
}

int check_small_m_args(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, const float *Y,
                       const char *who) {
    if (int rc = check_pack(w, who)) return rc;
    if (int rc = check_device(who)) return rc;
    if (M < 1 || M > 48) return fail(QVB8_ERR_ARG, "%s: M=%lld is outside 1..48", who, (long long)M);
    if (x_dtype != QVB8_F16 && x_dtype != QVB8_BF16 && x_dtype != QVB8_F32)
        return fail(QVB8_ERR_ARG, "%s: x_dtype %d is not QVB8_F16/BF16/F32", who, x_dtype);
    if (x_mode != 0 && x_mode != 1) return fail(QVB8_ERR_ARG, "%s: x_mode %d is not 0 or 1", who, x_mode);
    if ((!X && w->P > 0) || (!Y && w->Q > 0)) return fail(QVB8_ERR_ARG, "%s: null X or Y", who);
    return QVB8_OK;
}

}  // namespace qv

QV_API int qvb8_small_m_generic(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, float *Y,
                                void *stream) {
    using namespace qv;
    if (int rc = check_small_m_args(w, X, x_dtype, x_mode, M, Y, "qvb8_small_m_generic")) return rc;
    if (w->Q == 0) return QVB8_OK;
    return launch_small_m_generic(w, X, x_dtype, x_mode, (int)M, Y, reinterpret_cast<cudaStream_t>(stream));
}

QV_API const char *qvb8_last_error(void) { return qv::err_buf(); }

QV_API const char *qvb8_version(void) { return "qvb8_b200 0.1.0 (sm_100a)"; }
