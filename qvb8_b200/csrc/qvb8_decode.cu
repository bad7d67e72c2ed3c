// Dense restore of a QVB8 pack: W[q, c] = T(fma(id, tau_s[q], min_s[q])), one rounding to T, bit-exact with the
// reference decoder (formats/qvb8/decode.py:168-212; formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:535-699, 1711-1727).
//
// HBM-bound on the STORE side: 2 bytes written per ~0.8 bytes read.  One warp restores a 256-column segment of one
// row per step: a lane owns eight consecutive ids, which are exactly nb bytes of the row (rows are byte aligned when
// P % 8 == 0), fetched as three aligned 32-bit words; the eight results leave as one 16-byte store (32 for fp32), so
// a warp writes 512 contiguous bytes.  The grid is a fixed multiple of the SM count and strides over the segments.
// Built WITHOUT fast-math: the fused multiply-add and the narrowing are IEEE round-to-nearest-even.
#include "common.cuh"

namespace qv {

template <int NB, int J>
__device__ __forceinline__ uint32_t field_ct(uint32_t lo, uint32_t hi) {
    constexpr uint32_t MASK = (1u << NB) - 1u;
    constexpr int S = J * NB;
    if constexpr (S + NB <= 32) return (lo >> S) & MASK;
    else if constexpr (S >= 32) return (hi >> (S - 32)) & MASK;
    else return __funnelshift_r(lo, hi, S) & MASK;
}

template <int NB>
__device__ __forceinline__ void ids8_fixed(const uint8_t *__restrict__ ids, int64_t byte, uint32_t (&id)[8]) {
    const int64_t a0 = byte & ~(int64_t)3;
    const uint32_t *p = reinterpret_cast<const uint32_t *>(ids + a0);
    const uint32_t w0 = __ldg(p), w1 = __ldg(p + 1), w2 = __ldg(p + 2);
    const uint32_t sh = (uint32_t)(byte & 3) * 8u;
    const uint32_t lo = __funnelshift_r(w0, w1, sh), hi = __funnelshift_r(w1, w2, sh);
    id[0] = field_ct<NB, 0>(lo, hi); id[1] = field_ct<NB, 1>(lo, hi); id[2] = field_ct<NB, 2>(lo, hi);
    id[3] = field_ct<NB, 3>(lo, hi); id[4] = field_ct<NB, 4>(lo, hi); id[5] = field_ct<NB, 5>(lo, hi);
    id[6] = field_ct<NB, 6>(lo, hi); id[7] = field_ct<NB, 7>(lo, hi);
}

template <typename T> struct Store8;
template <> struct Store8<__half> {
    static __device__ __forceinline__ void go(__half *dst, const float (&v)[8]) {
        __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
        __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
        uint4 u;
        u.x = *reinterpret_cast<uint32_t *>(&a); u.y = *reinterpret_cast<uint32_t *>(&b);
        u.z = *reinterpret_cast<uint32_t *>(&c); u.w = *reinterpret_cast<uint32_t *>(&d);
        __stcs(reinterpret_cast<uint4 *>(dst), u);
    }
};
template <> struct Store8<__nv_bfloat16> {
    static __device__ __forceinline__ void go(__nv_bfloat16 *dst, const float (&v)[8]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
        uint4 u;
        u.x = *reinterpret_cast<uint32_t *>(&a); u.y = *reinterpret_cast<uint32_t *>(&b);
        u.z = *reinterpret_cast<uint32_t *>(&c); u.w = *reinterpret_cast<uint32_t *>(&d);
        __stcs(reinterpret_cast<uint4 *>(dst), u);
    }
};
template <> struct Store8<float> {
    static __device__ __forceinline__ void go(float *dst, const float (&v)[8]) {
        __stcs(reinterpret_cast<float4 *>(dst), make_float4(v[0], v[1], v[2], v[3]));
        __stcs(reinterpret_cast<float4 *>(dst) + 1, make_float4(v[4], v[5], v[6], v[7]));
    }
};

// Fast path: P % 8 == 0, ids 4-byte aligned, out 16-byte aligned.
template <typename T>
__global__ void __launch_bounds__(256) decode_rows_kernel(const uint8_t *__restrict__ ids, const float *__restrict__ min_s,
                                                          const float *__restrict__ tau_s,
                                                          const uint8_t *__restrict__ nbits,
                                                          const int64_t *__restrict__ bit_off, T *__restrict__ out,
                                                          int Q, int P) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int nseg = (P + 255) >> 8;
    const int64_t ntask = (int64_t)Q * nseg;
    for (int64_t task = warp; task < ntask; task += nwarps) {
        const int q = (int)(task / nseg);
        const int seg = (int)(task - (int64_t)q * nseg);
        const int c0 = seg * 256 + lane * 8;
        const int nb = __ldg(nbits + q);
        const int64_t base_bit = __ldg(bit_off + q);
        const float m = __ldg(min_s + q), ts = __ldg(tau_s + q);
        if (c0 >= P) continue;
        uint32_t id[8];
        const bool byte_row = (base_bit & 7) == 0;
        const int64_t byte = (base_bit >> 3) + (int64_t)(c0 >> 3) * nb;
        switch (byte_row ? nb : 0) {                       // warp-uniform
            case 4: ids8_fixed<4>(ids, byte, id); break;
            case 5: ids8_fixed<5>(ids, byte, id); break;
            case 6: ids8_fixed<6>(ids, byte, id); break;
            case 7: ids8_fixed<7>(ids, byte, id); break;
            case 8: ids8_fixed<8>(ids, byte, id); break;
            default:
#pragma unroll
                for (int j = 0; j < 8; ++j) id[j] = field_bytes(ids, base_bit + (int64_t)(c0 + j) * nb, nb);
        }
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmaf_rn(small_u2f(id[j]), ts, m);
        Store8<T>::go(out + (int64_t)q * P + c0, v);
    }
}

// Any layout: one element per thread.
template <typename T>
__global__ void __launch_bounds__(256) decode_elems_kernel(const uint8_t *__restrict__ ids, const float *__restrict__ min_s,
                                                           const float *__restrict__ tau_s,
                                                           const uint8_t *__restrict__ nbits,
                                                           const int64_t *__restrict__ bit_off, T *__restrict__ out,
                                                           int Q, int P) {
    const int64_t n = (int64_t)Q * P;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int q = (int)(i / P);
        const int c = (int)(i - (int64_t)q * P);
        const int nb = __ldg(nbits + q);
        const uint32_t id = field_bytes(ids, __ldg(bit_off + q) + (int64_t)c * nb, nb);
        out[i] = narrow<T>(__fmaf_rn(small_u2f(id), __ldg(tau_s + q), __ldg(min_s + q)));
    }
}

template <typename T>
__global__ void __launch_bounds__(256) scatter_escapes_kernel(const int64_t *__restrict__ esc_idx,
                                                              const float *__restrict__ esc_vals, int64_t n_esc,
                                                              int64_t n_out, T *__restrict__ out) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n_esc; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = __ldg(esc_idx + e);
        if (i >= 0 && i < n_out) out[i] = narrow<T>(__ldg(esc_vals + e));
    }
}

static int sm_count() {
    static thread_local int dev_cached = -1, n = 148;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != dev_cached) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        dev_cached = dev;
    }
    return n;
}

template <typename T>
static int decode_launch(const qvb8_pack *w, T *out, cudaStream_t st) {
    const int Q = (int)w->Q, P = (int)w->P;
    if (Q == 0 || P == 0) return QVB8_OK;
    const int sms = sm_count();
    const bool fast = (P % 8 == 0) && aligned(w->ids, 4) && aligned(out, 16);
    if (fast) {
        const int64_t ntask = (int64_t)Q * ((P + 255) / 256);
        const int64_t want = (ntask + 7) / 8;                         // 8 warps per block
        const int grid = (int)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);
        decode_rows_kernel<T><<<grid, 256, 0, st>>>(w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, out, Q, P);
    } else {
        const int64_t n = (int64_t)Q * P;
        const int64_t want = (n + 255) / 256;
        const int grid = (int)(want < (int64_t)sms * 16 ? want : (int64_t)sms * 16);
        decode_elems_kernel<T><<<grid, 256, 0, st>>>(w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, out, Q, P);
    }
    if (int rc = cuda_status("qvb8_decode launch")) return rc;
    if (w->n_esc > 0) {
        const int64_t want = (w->n_esc + 255) / 256;
        const int grid = (int)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);
        scatter_escapes_kernel<T><<<grid, 256, 0, st>>>(w->esc_idx, w->esc_vals, w->n_esc, (int64_t)Q * P, out);
        if (int rc = cuda_status("qvb8_decode escapes launch")) return rc;
    }
    return QVB8_OK;
}

// Row gather for embeddings: out[i, :] = restored row rows[i] (reference formats/qvb8/embedding.py:92-150
// QVBandEmbeddingV8._decode_rows + the escape loop of forward).  The reference computes min_s + id * tau_s with a
// multiplication and an addition (two roundings in fp32), not the fused multiply-add of the linear kernels, and then
// casts; the same two operations are used here so that the table is bit-identical.  One block per requested row; the
// row's escapes are found by binary search in the ascending flat indices.  A row index outside [0, Q) gives a row of
// zeros (the Python mirror checks the indices first, as torch's embedding does).
template <typename T>
__global__ void __launch_bounds__(256) embed_rows_kernel(const uint8_t *__restrict__ ids, const float *__restrict__ min_s,
                                                         const float *__restrict__ tau_s, const uint8_t *__restrict__ nbits,
                                                         const int64_t *__restrict__ bit_off, const int64_t *__restrict__ esc_idx,
                                                         const float *__restrict__ esc_vals, int64_t n_esc, int64_t Q, int P,
                                                         const int64_t *__restrict__ rows, T *__restrict__ out) {
    const int64_t i = blockIdx.x;
    const int64_t q = __ldg(rows + i);
    T *o = out + i * P;
    if (q < 0 || q >= Q) {
        for (int c = threadIdx.x; c < P; c += blockDim.x) o[c] = narrow<T>(0.f);
        return;
    }
    const int nb = __ldg(nbits + q);
    const int64_t b0 = __ldg(bit_off + q);
    const float ts = __ldg(tau_s + q), ms = __ldg(min_s + q);
    for (int c = threadIdx.x; c < P; c += blockDim.x)
        o[c] = narrow<T>(__fadd_rn(ms, __fmul_rn((float)field_bytes(ids, b0 + (int64_t)c * nb, nb), ts)));
    if (n_esc == 0) return;
    __syncthreads();
    // [lo, hi) = escapes with flat index in [q * P, (q + 1) * P)
    auto lower = [&](int64_t key) {
        int64_t a = 0, b = n_esc;
        while (a < b) {
            const int64_t m = (a + b) >> 1;
            if (__ldg(esc_idx + m) < key) a = m + 1; else b = m;
        }
        return a;
    };
    const int64_t lo = lower(q * P), hi = lower((q + 1) * P);
    for (int64_t e = lo + threadIdx.x; e < hi; e += blockDim.x) o[__ldg(esc_idx + e) - q * P] = narrow<T>(__ldg(esc_vals + e));
}

}  // namespace qv

QV_API int qvb8_decode(const qvb8_pack *w, int out_dtype, void *out, void *stream) {
    using namespace qv;
    if (int rc = check_pack(w, "qvb8_decode")) return rc;
    if (int rc = check_device("qvb8_decode")) return rc;
    if (!out && w->Q * w->P > 0) return fail(QVB8_ERR_ARG, "qvb8_decode: null output");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (out_dtype) {
        case QVB8_F16: return decode_launch<__half>(w, reinterpret_cast<__half *>(out), st);
        case QVB8_BF16: return decode_launch<__nv_bfloat16>(w, reinterpret_cast<__nv_bfloat16 *>(out), st);
        case QVB8_F32: return decode_launch<float>(w, reinterpret_cast<float *>(out), st);
        default: return fail(QVB8_ERR_ARG, "qvb8_decode: out_dtype %d is not QVB8_F16/BF16/F32", out_dtype);
    }
}

/* out (n, P) = the restored rows `rows[0 .. n)` (int64 device array) of the pack, escapes written over: the lookup of
 * an embedding table kept as a pack. */
QV_API int qvb8_embed_rows(const qvb8_pack *w, const int64_t *rows, int64_t n, int out_dtype, void *out, void *stream) {
    using namespace qv;
    if (int rc = check_pack(w, "qvb8_embed_rows")) return rc;
    if (int rc = check_device("qvb8_embed_rows")) return rc;
    if (n < 0 || n > 0x7fffffff || (n > 0 && (!rows || !out))) return fail(QVB8_ERR_ARG, "qvb8_embed_rows: bad rows / out / n");
    if (n == 0 || w->P == 0) return QVB8_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define QV_EMBED(T)                                                                                                   \
    embed_rows_kernel<T><<<(unsigned)n, 256, 0, st>>>(w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, w->esc_idx, \
                                                      w->esc_vals, w->n_esc, w->Q, (int)w->P, rows, reinterpret_cast<T *>(out))
    switch (out_dtype) {
        case QVB8_F16: QV_EMBED(__half); break;
        case QVB8_BF16: QV_EMBED(__nv_bfloat16); break;
        case QVB8_F32: QV_EMBED(float); break;
        default: return fail(QVB8_ERR_ARG, "qvb8_embed_rows: out_dtype %d is not QVB8_F16/BF16/F32", out_dtype);
    }
#undef QV_EMBED
    return cuda_status("qvb8_embed_rows");
}

// ---------------------------------------------------------------------------------------------------------------
// Greedy token choice over logits: per row of Y the largest value and the LOWEST index that holds it.  With the
// vocabulary split over ranks by output rows (the lm_head is the largest linear of a decoder) a rank reduces its own
// slice of the logits to one (value, index) pair per token, and the ranks exchange 16 bytes per token instead of their
// logits.  NaNs never win (a row of NaNs yields index_base and -inf).
namespace qv {

constexpr int ARGMAX_BLOCKS = 64;        // partial results per row
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t i) {
    // larger value first; among equal values the lower index: order-preserving float bits above, inverted index below
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - i);
}
__device__ __forceinline__ unsigned long long key_max(unsigned long long a, unsigned long long b) { return a > b ? a : b; }

__global__ void __launch_bounds__(256) argmax_partial_kernel(const float *__restrict__ Y, int64_t V, int64_t ldy,
                                                             unsigned long long *__restrict__ part) {
    const int m = blockIdx.y;
    const float *y = Y + (int64_t)m * ldy;
    const int64_t per = (V + gridDim.x - 1) / gridDim.x;
    const int64_t lo = (int64_t)blockIdx.x * per, hi = lo + per < V ? lo + per : V;
    unsigned long long best = argmax_key(-INFINITY, 0xffffffffu);       // below every real candidate
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = __ldg(y + i);
        if (v == v) best = key_max(best, argmax_key(v, (uint32_t)i));
    }
    for (int o = 16; o > 0; o >>= 1) best = key_max(best, __shfl_xor_sync(0xffffffffu, best, o));
    __shared__ unsigned long long s[8];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < 8; ++k) best = key_max(best, s[k]);
        part[(int64_t)m * gridDim.x + blockIdx.x] = best;
    }
}
__global__ void __launch_bounds__(32) argmax_final_kernel(const unsigned long long *__restrict__ part, int nblk,
                                                          int64_t index_base, float *__restrict__ best_val,
                                                          int64_t *__restrict__ best_idx) {
    const int m = blockIdx.x;
    unsigned long long best = argmax_key(-INFINITY, 0xffffffffu);
    for (int k = threadIdx.x; k < nblk; k += 32) best = key_max(best, part[(int64_t)m * nblk + k]);
    for (int o = 16; o > 0; o >>= 1) best = key_max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (threadIdx.x == 0) {
        uint32_t b = (uint32_t)(best >> 32);
        b = (b & 0x80000000u) ? (b & 0x7fffffffu) : ~b;
        const uint32_t i = 0xffffffffu - (uint32_t)(best & 0xffffffffu);
        const bool none = i == 0xffffffffu;                             // no candidate: every value was a NaN (or V = 0)
        best_val[m] = none ? -INFINITY : __uint_as_float(b);
        best_idx[m] = index_base + (none ? 0 : (int64_t)i);
    }
}

}  // namespace qv

QV_API int64_t qvb8_argmax_scratch_bytes(int64_t M) { return M > 0 ? M * qv::ARGMAX_BLOCKS * 8 : 0; }

/* best_val[m], best_idx[m] = the largest of Y[m, 0 .. V) (fp32, rows ldy apart) and index_base + the lowest column
 * that holds it; NaNs are passed over.  scratch: qvb8_argmax_scratch_bytes(M) bytes, 8-byte aligned. */
QV_API int qvb8_argmax_rows(const float *Y, int64_t M, int64_t V, int64_t ldy, int64_t index_base, float *best_val,
                            int64_t *best_idx, void *scratch, int64_t scratch_bytes, void *stream) {
    using namespace qv;
    if (int rc = check_device("qvb8_argmax_rows")) return rc;
    if (!Y || !best_val || !best_idx || M < 0 || M > 65535 || V < 0 || V >= 0xffffffffll || ldy < V)
        return fail(QVB8_ERR_ARG, "qvb8_argmax_rows: bad arguments");
    if (M == 0) return QVB8_OK;
    if (!scratch || scratch_bytes < qvb8_argmax_scratch_bytes(M) || !aligned(scratch, 8))
        return fail(QVB8_ERR_SCRATCH, "qvb8_argmax_rows: scratch of %lld bytes (8-byte aligned) needed",
                    (long long)qvb8_argmax_scratch_bytes(M));
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    unsigned long long *part = reinterpret_cast<unsigned long long *>(scratch);
    argmax_partial_kernel<<<dim3(ARGMAX_BLOCKS, (unsigned)M), 256, 0, st>>>(Y, V, ldy, part);
    if (int rc = cuda_status("qvb8_argmax_rows partial")) return rc;
    argmax_final_kernel<<<(unsigned)M, 32, 0, st>>>(part, ARGMAX_BLOCKS, index_base, best_val, best_idx);
    return cuda_status("qvb8_argmax_rows");
}
