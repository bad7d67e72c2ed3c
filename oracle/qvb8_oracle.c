/*
 * CPU oracle for the QVB8 / QVB8R fused decode-in-matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the reference's
 * pack-decoding algorithm so that the CUDA kernels can be checked against it.
 * Nothing in the shipped package may call into it: only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark load this library.
 *
 * Parity pin: the reference ships no tests, fixtures or known-answer vectors
 * for this path.  The oracle is pinned instead against outputs of the
 * reference's own code run on seeded packs and committed as golden fixtures
 * together with the scripts that produced them: for QVB8 its Python decoders
 * (formats/qvb8/decode.py, pack_container.py; tests/golden/make_golden.py),
 * for QVB8R files written by its container.py from streams coded by its C++
 * encode and decoded by its C++ embed_rows
 * (formats/qvb8r/backends/cuda_qvb8r/qvb8r_cpu.cpp;
 * tests/golden/make_golden_qvb8r.py).
 *
 * Every function cites the reference lines it follows (paths are relative to
 * the reference project root, under src/qv_band/).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* scalar helpers                                                            */

/* One NB-bit field starting at absolute bit `bit` of an LSB-first stream.
 * formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:46-55 (load_field) and
 * formats/qvb8/decode.py:317-343 (_unpack_bits_block): a field is at most 14
 * bits wide and so spans at most three bytes; the packer pads the payload with
 * eight zero bytes so reading four is always in bounds. */
static inline uint32_t field_at(const uint8_t *buf, int64_t bit, int nbits)
{
    const int64_t by = bit >> 3;
    const uint32_t sh = (uint32_t)(bit & 7);
    const uint32_t w = (uint32_t)buf[by] | ((uint32_t)buf[by + 1] << 8) |
                       ((uint32_t)buf[by + 2] << 16) | ((uint32_t)buf[by + 3] << 24);
    return (w >> sh) & ((1u << nbits) - 1u);
}

/* fp32 -> fp16 bits, round to nearest even, IEEE overflow to inf.
 * The reference narrows with numpy .astype(float16) (formats/qvb8/
 * backends_experts.py:70-72) and __float2half_rn (qvb8_cuda.cu:569-573). */
static inline uint16_t f32_to_f16_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x0200u | ((ax >> 13) & 0x3ffu) : 0u));
    if (ax >= 0x477ff000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    if (ax < 0x33000001u) /* < 2^-25 (or exactly 2^-25 ties to even 0) */
        return (uint16_t)sign;
    int e = (int)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    const uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    uint32_t r = base + q;
    if (rem > half || (rem == half && (q & 1u)))
        r += 1; /* carries into the exponent correctly */
    return (uint16_t)(sign | r);
}

/* fp32 -> bf16 bits, round to nearest even (torch .to(bfloat16);
 * __floats2bfloat162_rn at qvb8_cuda.cu:563-567). */
static inline uint16_t f32_to_bf16_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u)
        return (uint16_t)((x >> 16) | 0x0040u);
    const uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

static inline float f16_bits_to_f32(uint16_t h)
{
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu, x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else {
            int k = 0;
            while (!(m & 0x400u)) { m <<= 1; ++k; }
            x = sign | ((uint32_t)(127 - 15 - k + 1) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

static inline float bf16_bits_to_f32(uint16_t h)
{
    uint32_t x = (uint32_t)h << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* Saturating fp32 -> fp16 -> fp32 narrowing of an activation:
 * qvb8_cuda.cu:761-764 (sat_half): clamp to +-65504 by comparison (a NaN
 * passes through), then round to nearest even. */
static inline float sat_half_f32(float v)
{
    const float c = v > 65504.0f ? 65504.0f : (v < -65504.0f ? -65504.0f : v);
    return f16_bits_to_f32(f32_to_f16_bits(c));
}

/* ------------------------------------------------------------------------- */
/* QVB8: ids, restore, escapes                                               */

/* All ids of a pack, (Q, P) uint16.  formats/qvb8/decode.py:346-365
 * (unpack_bits_rows): row r occupies bits [bit_off[r], bit_off[r] +
 * nbits[r] * P), LSB-first, no padding between rows. */
ORACLE_API void qvb8o_unpack_ids(const uint8_t *buf, const uint8_t *nbits, const int64_t *bit_off,
                                 int64_t Q, int64_t P, uint16_t *ids)
{
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < Q; ++q) {
        const int nb = nbits[q];
        const int64_t base = bit_off[q];
        uint16_t *o = ids + q * P;
        for (int64_t c = 0; c < P; ++c)
            o[c] = (uint16_t)field_at(buf, base + c * nb, nb);
    }
}

/* Restored fp32 weights.  formats/qvb8/decode.py:168-212 (fma32 /
 * reconstruct): value = fma_rn((float)id, tau_s[q], min_s[q]) with a single
 * rounding, then the escapes overwrite their flat positions with the exact
 * stored value.  The CUDA side is fmaf at qvb8_cuda.cu:551. */
ORACLE_API void qvb8o_restore_f32(const uint16_t *ids, const float *min_s, const float *tau_s, int64_t Q,
                                  int64_t P, const int64_t *esc_idx, const float *esc_vals, int64_t n_esc,
                                  float *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < Q; ++q) {
        const float m = min_s[q], t = tau_s[q];
        const uint16_t *i = ids + q * P;
        float *o = out + q * P;
        for (int64_t c = 0; c < P; ++c)
            o[c] = fmaf((float)i[c], t, m);
    }
    for (int64_t e = 0; e < n_esc; ++e)
        out[esc_idx[e]] = esc_vals[e];
}

/* Dense restore straight from the packed payload to a 16-bit type, one
 * rounding of the fp32 band value; escapes are narrowed the same way and
 * written over their positions.  kind: 0 = fp16, 1 = bf16.
 * qvb8_cuda.cu:592-625 (decode kernel), :651-699 (fp16 + escape overwrite),
 * :1711-1727 (bf16). */
ORACLE_API void qvb8o_decode_16(const uint8_t *buf, const uint8_t *nbits, const int64_t *bit_off,
                                const float *min_s, const float *tau_s, int64_t Q, int64_t P,
                                const int64_t *esc_idx, const float *esc_vals, int64_t n_esc, int kind,
                                uint16_t *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < Q; ++q) {
        const int nb = nbits[q];
        const int64_t base = bit_off[q];
        const float m = min_s[q], t = tau_s[q];
        uint16_t *o = out + q * P;
        for (int64_t c = 0; c < P; ++c) {
            const float w = fmaf((float)field_at(buf, base + c * nb, nb), t, m);
            o[c] = kind ? f32_to_bf16_bits(w) : f32_to_f16_bits(w);
        }
    }
    for (int64_t e = 0; e < n_esc; ++e)
        out[esc_idx[e]] = kind ? f32_to_bf16_bits(esc_vals[e]) : f32_to_f16_bits(esc_vals[e]);
}

/* Small-M product Y[m, q] = sum_c X[m, c] * W[q, c] the way the reference
 * GEMV defines it: the activation is first narrowed to saturated fp16
 * (qvb8_cuda.cu:1082, :1102), the weight is the un-narrowed fp32 band value
 * (:346-353) or, at an escaped position, the exact stored value (:507-533).
 * Accumulated in double here so the oracle itself adds no rounding; the GPU
 * result is compared with a tolerance.  narrow_x: 1 = saturating fp16 (QVB8),
 * 0 = keep fp32 (QVB8R keeps X in fp32 for M <= 8, qvb8r/module.py:210-220). */
ORACLE_API void qvb8o_matmul_f32w(const float *X, int64_t M, const float *W, int64_t Q, int64_t P,
                                  int narrow_x, double *Y)
{
    float *Xn = (float *)malloc((size_t)M * P * sizeof(float));
    for (int64_t i = 0; i < M * P; ++i)
        Xn[i] = narrow_x ? sat_half_f32(X[i]) : X[i];
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < Q; ++q) {
        const float *w = W + q * P;
        for (int64_t m = 0; m < M; ++m) {
            const float *x = Xn + m * P;
            double a = 0.0;
            for (int64_t c = 0; c < P; ++c)
                a += (double)x[c] * (double)w[c];
            Y[m * Q + q] = a;
        }
    }
    free(Xn);
}

/* Element-wise narrowing helpers exported for the Python side of the oracle. */
ORACLE_API void qvb8o_f32_to_f16(const float *in, int64_t n, uint16_t *out)
{
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_f16_bits(in[i]);
}
ORACLE_API void qvb8o_f32_to_bf16(const float *in, int64_t n, uint16_t *out)
{
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16_bits(in[i]);
}
ORACLE_API void qvb8o_sat_half(const float *in, int64_t n, float *out)
{
    for (int64_t i = 0; i < n; ++i) out[i] = sat_half_f32(in[i]);
}

/* ------------------------------------------------------------------------- */
/* QVB8R: rANS tile walk                                                     */

/* All ids of a .qvb8r tensor, (Q, P) int16, rows at their ORIGINAL index.
 *
 * formats/qvb8r/backends/cuda_qvb8r/qvb8r_cpu.cpp:13-58 (embed_rows) and
 * qvb8r_cuda.cu:36-75 (Stream): a tile holds `rows` consecutive sorted rows of
 * one class and 32 interleaved 64-bit rANS states.  State j decodes column
 * 32*step + j.  Per symbol E = tab[class][x & 4095]; s = E & 2047;
 * x = ((E >> 22) + 1) * (x >> 12) + ((E >> 11) & 2047).  Symbols go in pairs:
 * after a lane decoded two, a state below 2^32 takes the tile's next 32-bit
 * word, lanes in ascending order (the order the GPU ballot hands words out).
 * id = s + drow[row] (rows are coded centred, codec.py:4-9).
 *
 *   tiles    (nt, 3) int64: class, first sorted row, rows
 *   tile_off (nt + 1) int64 word offsets
 *   states   (nt, 32) uint64
 *   tab      (K, 4096) uint32 slot tables (codec.py:11-20 slot_tables)
 *   perm     (Q) int32 sorted row -> original row
 *   drow     (Q) int32 by original row
 * Returns 0, or -1 if a tile would read past n_words. */
/* one decoding step of a lane: looks the state's low 12 bits up in the class's slot table, returns the symbol and
 * advances the state to freq * (state >> 12) + offset_in_symbol (qvb8r_cpu.cpp:41-43; entry layout codec.py:19) */
static inline int rans_step(const uint32_t *slot, uint64_t *state)
{
    const uint32_t entry = slot[*state & 4095u];
    const uint64_t freq = (uint64_t)(entry >> 22) + 1u, within = (entry >> 11) & 2047u;
    *state = freq * (*state >> 12) + within;
    return (int)(entry & 2047u);
}

ORACLE_API int qvb8ro_decode_ids(const uint32_t *words, int64_t n_words, const int64_t *tile_off,
                                 const uint64_t *states, const int64_t *tiles, int64_t nt,
                                 const uint32_t *tab, const int32_t *perm, const int32_t *drow, int64_t P,
                                 int16_t *ids)
{
    const int64_t pairs = P / 64;            /* a lane decodes two symbols (columns 64 k + lane, 64 k + 32 + lane) per visit */
    int overrun = 0;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t t = 0; t < nt; ++t) {
        const uint32_t *slot = tab + tiles[3 * t] * 4096;
        const int64_t first = tiles[3 * t + 1], rows = tiles[3 * t + 2];
        uint64_t lane_state[32];
        memcpy(lane_state, states + t * 32, sizeof lane_state);
        int64_t next_word = tile_off[t];
        for (int64_t r = 0; r < rows; ++r) {
            const int32_t q = perm[first + r];
            int16_t *row = ids + (int64_t)q * P;
            for (int64_t k = 0; k < pairs; ++k) {
                for (int lane = 0; lane < 32; ++lane) {          /* ascending lanes: the order words are handed out in */
                    uint64_t st = lane_state[lane];
                    row[64 * k + lane] = (int16_t)(rans_step(slot, &st) + drow[q]);
                    row[64 * k + 32 + lane] = (int16_t)(rans_step(slot, &st) + drow[q]);
                    if (st < (1ull << 32)) {                      /* renormalise: take the tile's next 32-bit word */
                        uint32_t w = 0;
                        if (next_word < n_words) w = words[next_word++];
                        else overrun = 1;
                        st = (st << 32) | w;
                    }
                    lane_state[lane] = st;
                }
            }
        }
    }
    return overrun ? -1 : 0;
}

/* Band value of signed ids (QVB8R ids can be offset by drow): the GPU kernels
 * use fmaf (qvb8r_cuda.cu:10, :114) -- NOT the mul-then-add of the CPU
 * embedding reader (qvb8r_cpu.cpp:44), which differs by one ulp in places. */
ORACLE_API void qvb8ro_restore_f32(const int16_t *ids, const float *min_s, const float *tau_s, int64_t Q,
                                   int64_t P, float *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < Q; ++q) {
        const float m = min_s[q], t = tau_s[q];
        for (int64_t c = 0; c < P; ++c)
            out[q * P + c] = fmaf((float)ids[q * P + c], t, m);
    }
}

ORACLE_API int qvb8o_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
