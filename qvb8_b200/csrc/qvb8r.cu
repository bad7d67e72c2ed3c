// QVB8R (entropy-coded QVB8) for sm_100a: ids, dense restore and small-M products straight from the rANS stream.
//
// Replaces the reference's qvb8r_cuda kernels (formats/qvb8r/backends/cuda_qvb8r/qvb8r_cuda.cu:36-75 stream,
// :85-270 gemv / multi / tc, :272-308 decode, :310-320 fix_escapes).  The format (container.py:1-12, codec.py:4-21):
// rows sorted by class; a tile = a few consecutive sorted rows of one class coded by 32 interleaved 64-bit rANS
// states; state j codes column 32 * step + j; per symbol  E = tab[class][x & 4095],  s = E & 2047,
// x = ((E >> 22) + 1) * (x >> 12) + ((E >> 11) & 2047);  symbols go in pairs and after a pair every state below
// 2^32 takes the tile's next 32-bit word, lanes in ascending order; id = s + drow[row]; w = fma(id, tau_s, min_s).
//
// This is integer work with a serial dependency per state, so it is bound by instruction latency and issue, not by
// HBM (the stream is ~5 bits per weight); what a B200 offers it is many resident warps.  One warp walks one tile
// (lane j = state j), eight tiles of one class per CTA share the class's 16 KB slot table in shared memory.  The
// word stream is read through a 64-word register window (two coalesced 128-byte loads always in flight ahead of
// the cursor) and handed to the lanes that refill with a ballot, a popcount and two shuffles: no shared-memory ring,
// no dependent global load on the decode chain.
//
// Products follow the reference's contracts: `gemv` / `multi` multiply the fp32 band value with fp32 X (bf16 X is
// exact in fp32); `tc` rounds the band value once to fp16 and multiplies fp16 X, fp32 accumulation.  Every row sum is
// a fixed-order lane sum: results are identical from run to run.  Escapes are corrected afterwards from their stored
// differences, one thread per (token, output) in stored order (:310-320).
#include "common.cuh"

namespace qv {

constexpr int R_WPB = 8;                   // warps = tiles per CTA (a block of the schedule holds at most this many)

struct RStream {
    uint64_t x;
    uint32_t w0, w1;                       // words [cursor .. cursor + 64) of the tile's stream, lane-striped
    int c;                                 // words of the window already consumed (< 32)
    const uint32_t *next;                  // the words after the window
};

__device__ __forceinline__ void rstream_init(RStream &z, const uint32_t *__restrict__ words, int64_t off,
                                             const uint64_t *__restrict__ states, int tile, int lane) {
    const uint32_t *p = words + off;
    z.x = __ldg(states + (int64_t)tile * 32 + lane);
    z.w0 = __ldg(p + lane);
    z.w1 = __ldg(p + 32 + lane);
    z.c = 0;
    z.next = p + 64;
}

// Two symbols per lane, then the refill.
__device__ __forceinline__ void rstream_pair(RStream &z, const uint32_t *st, int lane, uint32_t &s1, uint32_t &s2) {
    uint32_t E = st[(uint32_t)z.x & 4095u];
    s1 = E & 2047u;
    z.x = (uint64_t)((E >> 22) + 1u) * (z.x >> 12) + ((E >> 11) & 2047u);
    E = st[(uint32_t)z.x & 4095u];
    s2 = E & 2047u;
    z.x = (uint64_t)((E >> 22) + 1u) * (z.x >> 12) + ((E >> 11) & 2047u);
    const bool need = z.x < (1ull << 32);
    const uint32_t mask = __ballot_sync(0xffffffffu, need);
    const int idx = z.c + __popc(mask & ((1u << lane) - 1u));
    const uint32_t v0 = __shfl_sync(0xffffffffu, z.w0, idx & 31), v1 = __shfl_sync(0xffffffffu, z.w1, idx & 31);
    if (need) z.x = (z.x << 32) | (idx < 32 ? v0 : v1);
    z.c += __popc(mask);
    if (z.c >= 32) {                       // uniform over the warp
        z.w0 = z.w1;
        z.w1 = __ldg(z.next + lane);
        z.next += 32;
        z.c -= 32;
    }
}

struct RCore {
    const uint32_t *words;
    const int64_t *tile_off;
    const uint64_t *states;
    const int64_t *tiles;                  // (nt, 3): class, first sorted row, rows
    const int32_t *blocks;                 // (nb, 3): class, first tile, tiles (<= R_WPB)
    const uint32_t *tab;                   // (K, 4096)
    const int32_t *perm;                   // sorted row -> original row
    const float *min_s, *tau_s;            // by original row
    const int32_t *drow;                   // by original row
    int Q, P;
};

// MODE 0: ids (int16).  MODE 1: dense restore to OutT.  MODE 2: products with MP tokens of XT; WROUND: round the band
// value to fp16 first (the reference's tensor-core contract).
template <int MODE, typename OutT, int MP, typename XT, bool WROUND>
__global__ void __launch_bounds__(32 * R_WPB) qvb8r_kernel(const RCore c, int b0, int64_t row_base, OutT *__restrict__ out,
                                                          const XT *__restrict__ X, int M, float *__restrict__ Y) {
    __shared__ uint32_t st[4096];
    const int32_t *blk = c.blocks + 3 * (int64_t)(b0 + blockIdx.x);
    const int cls = blk[0], tb = blk[1], ntb = blk[2];
    for (int i = threadIdx.x; i < 4096; i += blockDim.x) st[i] = __ldg(c.tab + (int64_t)cls * 4096 + i);
    __syncthreads();
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (w >= ntb) return;
    const int tile = tb + w;
    const int r0 = (int)c.tiles[3 * (int64_t)tile + 1], nr = (int)c.tiles[3 * (int64_t)tile + 2];
    const int S = c.P / 32;
    RStream z;
    rstream_init(z, c.words, c.tile_off[tile], c.states, tile, lane);
    for (int r = 0; r < nr; ++r) {
        const int orow = c.perm[r0 + r];
        const float m = c.min_s[orow], t = c.tau_s[orow];
        const int dr = c.drow[orow];
        float acc[MP];
#pragma unroll
        for (int k = 0; k < MP; ++k) acc[k] = 0.f;
        const int64_t orow_out = row_base < 0 ? (int64_t)orow : (int64_t)(r0 + r) - row_base;
        // the activations of a step are fetched one step ahead: their latency hides behind the decoder's dependency chain
        constexpr bool AHEAD = MODE == 2 && MP <= 8;       // beyond 8 tokens the extra registers cost more than they hide
        float xa[MP], xb[MP];
        if constexpr (AHEAD) {
#pragma unroll
            for (int k = 0; k < MP; ++k) {
                xa[k] = k < M ? (float)X[(int64_t)k * c.P + lane] : 0.f;
                xb[k] = k < M ? (float)X[(int64_t)k * c.P + lane + 32] : 0.f;
            }
        }
        for (int s0 = 0; s0 < S; s0 += 2) {
            float na[MP], nb_[MP];
            if constexpr (AHEAD) {
                const int cn = min(s0 + 2, S - 2) * 32 + lane;
#pragma unroll
                for (int k = 0; k < MP; ++k) {
                    na[k] = k < M ? (float)X[(int64_t)k * c.P + cn] : 0.f;
                    nb_[k] = k < M ? (float)X[(int64_t)k * c.P + cn + 32] : 0.f;
                }
            }
            uint32_t s1, s2;
            rstream_pair(z, st, lane, s1, s2);
            const int i1 = (int)s1 + dr, i2 = (int)s2 + dr;
            const int c1 = s0 * 32 + lane, c2 = c1 + 32;
            if constexpr (MODE == 0) {
                reinterpret_cast<int16_t *>(out)[orow_out * c.P + c1] = (int16_t)i1;
                reinterpret_cast<int16_t *>(out)[orow_out * c.P + c2] = (int16_t)i2;
            } else {
                float w1 = __fmaf_rn((float)i1, t, m), w2 = __fmaf_rn((float)i2, t, m);
                if constexpr (MODE == 1) {
                    out[orow_out * c.P + c1] = narrow<OutT>(w1);
                    out[orow_out * c.P + c2] = narrow<OutT>(w2);
                } else {
                    if (WROUND) { w1 = __half2float(__float2half_rn(w1)); w2 = __half2float(__float2half_rn(w2)); }
#pragma unroll
                    for (int k = 0; k < MP; ++k) {
                        if constexpr (AHEAD) {
                            acc[k] = __fmaf_rn(xa[k], w1, acc[k]);
                            acc[k] = __fmaf_rn(xb[k], w2, acc[k]);
                            xa[k] = na[k];
                            xb[k] = nb_[k];
                        } else if (k < M) {
                            acc[k] = __fmaf_rn((float)X[(int64_t)k * c.P + c1], w1, acc[k]);
                            acc[k] = __fmaf_rn((float)X[(int64_t)k * c.P + c2], w2, acc[k]);
                        }
                    }
                }
            }
        }
        if constexpr (MODE == 2) {
#pragma unroll
            for (int k = 0; k < MP; ++k) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
                if (lane == 0 && k < M) Y[(int64_t)k * c.Q + orow] = acc[k];
            }
        }
    }
}

// Y[m, uq[u]] += sum_e x[m, ec[e]] * ed[e], e in [ptr[u], ptr[u + 1]) in stored order (qvb8r_cuda.cu:310-320)
__global__ void __launch_bounds__(128) qvb8r_fix_kernel(const float *__restrict__ X, const int64_t *__restrict__ uq,
                                                        const int64_t *__restrict__ ptr, const int64_t *__restrict__ ec,
                                                        const float *__restrict__ ed, float *__restrict__ Y, int64_t U, int M,
                                                        int P, int Q) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= U * M) return;
    const int64_t u = i % U;
    const int m = (int)(i / U);
    const float *x = X + (int64_t)m * P;
    float a = 0.f;
    for (int64_t e = ptr[u]; e < ptr[u + 1]; ++e) a = __fmaf_rn(x[ec[e]], ed[e], a);
    Y[(int64_t)m * Q + uq[u]] += a;
}

// Embedding lookup: out[i, :] = row rows[i] of the table, restored as the reference's CPU reader restores it -- a
// multiplication and then an addition, min_s + float(id) * tau_s, not fused (qvb8r_cpu.cpp:44) -- with the row's escapes
// written over.  One warp per requested row: it walks the row's tile from the tile's start (a tile is a few rows) and
// keeps only the last row it decodes.  The slot table is read through the read-only cache: the warps of a CTA need
// different classes, and a lookup touches a handful of rows.
__global__ void __launch_bounds__(32 * R_WPB) qvb8r_embed_kernel(const RCore c, const int64_t *__restrict__ rows, int64_t n,
                                                                const int32_t *__restrict__ inv_perm,
                                                                const int32_t *__restrict__ row_tile,
                                                                const int64_t *__restrict__ esc_ptr,
                                                                const int32_t *__restrict__ esc_col,
                                                                const float *__restrict__ esc_val, float *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * R_WPB + (threadIdx.x >> 5);
    if (i >= n) return;
    const int64_t q = rows[i];
    float *o = out + i * c.P;
    if (q < 0 || q >= c.Q) {                                           // refused on the host; never read out of range
        for (int col = lane; col < c.P; col += 32) o[col] = 0.f;
        return;
    }
    const int sp = inv_perm[q], tile = row_tile[sp];
    const int k = sp - (int)c.tiles[3 * (int64_t)tile + 1];            // rows of the tile in front of this one
    const uint32_t *st = c.tab + c.tiles[3 * (int64_t)tile] * 4096;
    const float m = c.min_s[q], t = c.tau_s[q];
    const int dr = c.drow[q];
    const int S = c.P / 32;
    RStream z;
    rstream_init(z, c.words, c.tile_off[tile], c.states, tile, lane);
    for (int r = 0; r <= k; ++r)
        for (int s0 = 0; s0 < S; s0 += 2) {
            uint32_t s1, s2;
            rstream_pair(z, st, lane, s1, s2);
            if (r == k) {
                o[s0 * 32 + lane] = __fadd_rn(m, __fmul_rn((float)((int)s1 + dr), t));
                o[s0 * 32 + 32 + lane] = __fadd_rn(m, __fmul_rn((float)((int)s2 + dr), t));
            }
        }
    __syncwarp();
    for (int64_t e = esc_ptr[q] + lane; e < esc_ptr[q + 1]; e += 32) o[esc_col[e]] = esc_val[e];
}

static int check_rpack(const qvb8r_pack *w, const char *who) {
    if (!w) return fail(QVB8_ERR_ARG, "%s: null pack", who);
    if (!w->words || !w->tile_off || !w->states || !w->tiles || !w->blocks || !w->tab || !w->perm || !w->min_s ||
        !w->tau_s || !w->drow)
        return fail(QVB8_ERR_ARG, "%s: null core array", who);
    if (w->Q <= 0 || w->P <= 0 || w->Q > 0x7fffffff || w->P > 0x7fffffff || w->P % 64 != 0)
        return fail(QVB8_ERR_ARG, "%s: Q=%lld P=%lld (P must be a multiple of 64)", who, (long long)w->Q, (long long)w->P);
    if (w->n_blocks < 0 || w->n_tiles < 0 || w->n_blocks > 0x7fffffff)
        return fail(QVB8_ERR_ARG, "%s: bad tile / block counts", who);
    return QVB8_OK;
}
static RCore core_of(const qvb8r_pack *w) {
    return RCore{w->words, w->tile_off, w->states, w->tiles, w->blocks, w->tab, w->perm, w->min_s, w->tau_s, w->drow,
                 (int)w->Q, (int)w->P};
}

template <int MP, typename XT, bool WROUND>
static void launch_mm(const RCore &c, int nb, const void *X, int M, float *Y, cudaStream_t st) {
    qvb8r_kernel<2, float, MP, XT, WROUND><<<nb, 32 * R_WPB, 0, st>>>(c, 0, -1, nullptr, reinterpret_cast<const XT *>(X), M, Y);
}
template <typename XT, bool WROUND>
static void launch_mm_mp(const RCore &c, int nb, const void *X, int M, float *Y, cudaStream_t st) {
    if (M <= 1) launch_mm<1, XT, WROUND>(c, nb, X, M, Y, st);
    else if (M <= 2) launch_mm<2, XT, WROUND>(c, nb, X, M, Y, st);
    else if (M <= 4) launch_mm<4, XT, WROUND>(c, nb, X, M, Y, st);
    else if (M <= 8) launch_mm<8, XT, WROUND>(c, nb, X, M, Y, st);
    else launch_mm<16, XT, WROUND>(c, nb, X, M, Y, st);
}

}  // namespace qv

QV_API int qvb8r_ids(const qvb8r_pack *w, int16_t *out, void *stream) {
    using namespace qv;
    if (int rc = check_rpack(w, "qvb8r_ids")) return rc;
    if (int rc = check_device("qvb8r_ids")) return rc;
    if (!out) return fail(QVB8_ERR_ARG, "qvb8r_ids: null output");
    if (w->n_blocks == 0) return QVB8_OK;
    qvb8r_kernel<0, int16_t, 1, float, false><<<(unsigned)w->n_blocks, 32 * R_WPB, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        core_of(w), 0, -1, out, nullptr, 0, nullptr);
    return cuda_status("qvb8r_ids");
}

QV_API int qvb8r_decode(const qvb8r_pack *w, int out_dtype, void *out, int64_t b0, int64_t nb, int64_t row_base,
                        void *stream) {
    using namespace qv;
    if (int rc = check_rpack(w, "qvb8r_decode")) return rc;
    if (int rc = check_device("qvb8r_decode")) return rc;
    if (!out) return fail(QVB8_ERR_ARG, "qvb8r_decode: null output");
    if (b0 < 0 || nb < 0 || b0 + nb > w->n_blocks) return fail(QVB8_ERR_ARG, "qvb8r_decode: block range out of bounds");
    if (nb == 0) return QVB8_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const RCore c = core_of(w);
    if (out_dtype == QVB8_F16)
        qvb8r_kernel<1, __half, 1, float, false><<<(unsigned)nb, 32 * R_WPB, 0, st>>>(c, (int)b0, row_base, reinterpret_cast<__half *>(out), nullptr, 0, nullptr);
    else if (out_dtype == QVB8_BF16)
        qvb8r_kernel<1, __nv_bfloat16, 1, float, false><<<(unsigned)nb, 32 * R_WPB, 0, st>>>(c, (int)b0, row_base, reinterpret_cast<__nv_bfloat16 *>(out), nullptr, 0, nullptr);
    else if (out_dtype == QVB8_F32)
        qvb8r_kernel<1, float, 1, float, false><<<(unsigned)nb, 32 * R_WPB, 0, st>>>(c, (int)b0, row_base, reinterpret_cast<float *>(out), nullptr, 0, nullptr);
    else
        return fail(QVB8_ERR_ARG, "qvb8r_decode: bad output dtype");
    return cuda_status("qvb8r_decode");
}

QV_API int qvb8r_small_m(const qvb8r_pack *w, const void *X, int x_dtype, int64_t M, int round_w_fp16, float *Y,
                         void *stream) {
    using namespace qv;
    if (int rc = check_rpack(w, "qvb8r_small_m")) return rc;
    if (int rc = check_device("qvb8r_small_m")) return rc;
    if (!X || !Y) return fail(QVB8_ERR_ARG, "qvb8r_small_m: null argument");
    if (M < 1 || M > 16) return fail(QVB8_ERR_ARG, "qvb8r_small_m: M=%lld is outside 1..16", (long long)M);
    if (w->n_blocks == 0) return QVB8_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const RCore c = core_of(w);
    const int nb = (int)w->n_blocks;
    if (x_dtype == QVB8_F32) {
        if (round_w_fp16) launch_mm_mp<float, true>(c, nb, X, (int)M, Y, st); else launch_mm_mp<float, false>(c, nb, X, (int)M, Y, st);
    } else if (x_dtype == QVB8_BF16) {
        if (round_w_fp16) launch_mm_mp<__nv_bfloat16, true>(c, nb, X, (int)M, Y, st); else launch_mm_mp<__nv_bfloat16, false>(c, nb, X, (int)M, Y, st);
    } else if (x_dtype == QVB8_F16) {
        if (round_w_fp16) launch_mm_mp<__half, true>(c, nb, X, (int)M, Y, st); else launch_mm_mp<__half, false>(c, nb, X, (int)M, Y, st);
    } else {
        return fail(QVB8_ERR_ARG, "qvb8r_small_m: bad X dtype");
    }
    return cuda_status("qvb8r_small_m");
}

QV_API int qvb8r_fix_escapes(const float *X, const int64_t *uq, const int64_t *ptr, const int64_t *ec, const float *ed,
                             float *Y, int64_t U, int64_t M, int64_t P, int64_t Q, void *stream) {
    using namespace qv;
    if (int rc = check_device("qvb8r_fix_escapes")) return rc;
    if (U == 0) return QVB8_OK;
    if (!X || !uq || !ptr || !ec || !ed || !Y || U < 0 || M <= 0 || P <= 0 || Q <= 0)
        return fail(QVB8_ERR_ARG, "qvb8r_fix_escapes: bad argument");
    const int64_t n = U * M;
    qvb8r_fix_kernel<<<(unsigned)((n + 127) / 128), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(X, uq, ptr, ec, ed, Y, U,
                                                                                                      (int)M, (int)P, (int)Q);
    return cuda_status("qvb8r_fix_escapes");
}

QV_API int qvb8r_embed_rows(const qvb8r_pack *w, const int64_t *rows, int64_t n, const int32_t *inv_perm,
                            const int32_t *row_tile, const int64_t *esc_ptr, const int32_t *esc_col, const float *esc_val,
                            float *out, void *stream) {
    using namespace qv;
    if (int rc = check_rpack(w, "qvb8r_embed_rows")) return rc;
    if (int rc = check_device("qvb8r_embed_rows")) return rc;
    if (n == 0) return QVB8_OK;
    if (!rows || !inv_perm || !row_tile || !esc_ptr || !out || n < 0)
        return fail(QVB8_ERR_ARG, "qvb8r_embed_rows: bad argument");
    qvb8r_embed_kernel<<<(unsigned)((n + R_WPB - 1) / R_WPB), 32 * R_WPB, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        core_of(w), rows, n, inv_perm, row_tile, esc_ptr, esc_col, esc_val, out);
    return cuda_status("qvb8r_embed_rows");
}
