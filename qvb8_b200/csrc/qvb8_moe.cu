// QVB8 mixture-of-experts MLP for a handful of tokens (decode / verify): out[t] = sum_j w[t,j] * down_e( act( up_e(x_t) ) ),
// e = idx[t,j], over stacked expert packs.
//
// Replaces the reference's fused expert stack (formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:844-992 gated SiLU,
// :994-1058 relu^2; stacked layout built by formats/qvb8/backends_experts.py:144-196).  The reference makes every
// (token, expert) PAIR one row block of a grouped GEMV, so an expert chosen by several tokens is read once per
// token.  Here the pairs are first grouped by expert (one small kernel, deterministic), and every selected expert's
// rows are then streamed ONCE for all the tokens that chose it: the bytes read are those of the distinct experts.
//
// Four launches: route -> up (+ activation) -> down -> combine.  HBM roofline: bytes = sum over distinct selected
// experts of their up and down rows.  A warp owns one output row (for the gated form: gate row i and up row I + i
// together, so the activation is applied in registers and the pre-activation never goes to memory); each lane takes 8
// consecutive columns of a 256-column block, which are exactly nb whole bytes; the row sum is reduced with shuffles.
// Arithmetic as the reference's GEMV: fp32 band value fma(id, tau_s, min_s), fp32 FMA accumulation; X narrowed to
// saturated fp16 first (qvb8_cuda.cu:1069, saturating_half), the hidden activations stay fp32.
#include "common.cuh"

namespace qv {

constexpr int MOE_WARPS = 8;
constexpr int MOE_TOK = 4;                 // tokens per pass over a row

struct MoeRoute {                          // device tables built by the route kernel
    int *counts;                           // [E] pairs that chose expert e
    int *lists;                            // [E][M] their pair numbers p = t * topk + j, ascending
    int *slots;                            // [min(E, npairs)] the distinct chosen experts, ascending
    int *nslots;                           // [1]
    int *bad;                              // [1] set when a pair could not be listed (see valid)
    int *valid;                            // [npairs] 1 = the pair is in its expert's list; 0 = its expert index is outside
                                           // [0, E), or the token named one expert more than M times: the pair's rows
                                           // are never computed and the combine step counts them as zero
};

// Block 0: thread e scans the pairs for expert e (at most a few hundred pairs): deterministic, no atomics.
// Blocks 1..: the activations once as fp32 values of their saturated-fp16 narrowing (what every row product reads,
// qvb8_cuda.cu:963 `saturating_half(X).to(float)`).
__global__ void __launch_bounds__(256) moe_route_kernel(const int64_t *__restrict__ idx, int npairs, int E, int M,
                                                        MoeRoute r, const void *__restrict__ X, int x_dtype, int64_t nx,
                                                        float *__restrict__ Xf) {
    if (blockIdx.x > 0) {
        for (int64_t i = (int64_t)(blockIdx.x - 1) * blockDim.x + threadIdx.x; i < nx; i += (int64_t)(gridDim.x - 1) * blockDim.x) {
            const float v = x_dtype == QVB8_F32 ? __ldg(reinterpret_cast<const float *>(X) + i)
                          : x_dtype == QVB8_BF16 ? __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16 *>(X) + i))
                                                 : __half2float(__ldg(reinterpret_cast<const __half *>(X) + i));
            Xf[i] = __half2float(sat_half(v));
        }
        return;
    }
    __shared__ int any_bad;
    if (threadIdx.x == 0) any_bad = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < npairs; p += blockDim.x) {
        const int64_t e = idx[p];
        if (e < 0 || e >= E) any_bad = 1;
        r.valid[p] = 0;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int p = 0; p < npairs; ++p)
            if (idx[p] == e) {
                if (c < M) { r.lists[(size_t)e * M + c++] = p; r.valid[p] = 1; }
                else any_bad = 1;
            }
        r.counts[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int n = 0;
        for (int e = 0; e < E; ++e)
            if (r.counts[e] > 0) r.slots[n++] = e;
        *r.nslots = n;
        *r.bad = any_bad;
    }
}

struct MoeRows {
    const float *X;            // ACT 0/1: (M, P) narrowed activations, by token; ACT 2: (npairs, P) hidden, by pair
    int topk;
    const uint8_t *ids;
    const float *min_s, *tau_s;   // [E][Q]
    const uint8_t *nbits;
    const int64_t *bit_off;       // global bit offsets into ids
    int Q, P;                     // rows per expert, columns
    int R;                        // outputs per pair: ACT 0: Q / 2, else Q
    float *out;                   // (npairs, R) fp32
    MoeRoute route;
    int M;
};

// 8 ids of width nb (<= 8) that start at byte `a` of the stream: exactly nb bytes, fetched as two aligned 8-byte words
// (the stream carries pad bytes after its last row).
__device__ __forceinline__ uint64_t load_8_fields(const uint8_t *__restrict__ ids, int64_t a) {
    const uint64_t *w = reinterpret_cast<const uint64_t *>(ids + (a & ~(int64_t)7));
    const uint64_t lo = __ldg(w), hi = __ldg(w + 1);
    const int sh = (int)(a & 7) * 8;
    return sh ? (lo >> sh) | (hi << (64 - sh)) : lo;
}

__device__ __forceinline__ void load_x8(const float *__restrict__ X, int64_t off, float (&x)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(X + off));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(X + off) + 1);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// ACT: 0 = gated SiLU (rows i and I + i of the up pack -> H[p, i] = silu(g) * u), 1 = relu^2 (row i -> H[p, i]),
// 2 = none (row d of the down pack, X by pair -> Y[p, d]).
struct MoeRowMeta {
    int nb;
    int64_t bit0;
    float ms, ts;
};
__device__ __forceinline__ MoeRowMeta moe_row_meta(const MoeRows &p, size_t mi) {
    MoeRowMeta m;
    m.nb = __ldg(p.nbits + mi);
    m.bit0 = __ldg(p.bit_off + mi);
    m.ms = __ldg(p.min_s + mi);
    m.ts = __ldg(p.tau_s + mi);
    return m;
}

template <int ACT>
__global__ void __launch_bounds__(MOE_WARPS * 32, 4) moe_rows_kernel(const MoeRows p) {
    const int s = blockIdx.y;
    if (s >= *p.route.nslots) return;
    const int e = p.route.slots[s];
    const int c = p.route.counts[e];
    const int *plist = p.route.lists + (size_t)e * p.M;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wstride = gridDim.x * MOE_WARPS;
    constexpr int NR = ACT == 0 ? 2 : 1;
    int r = blockIdx.x * MOE_WARPS + warp;
    if (r >= p.R) return;
    MoeRowMeta nxt[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) nxt[k] = moe_row_meta(p, (size_t)e * p.Q + r + (size_t)k * p.R);
    for (; r < p.R; r += wstride) {
        MoeRowMeta m[NR];
#pragma unroll
        for (int k = 0; k < NR; ++k) m[k] = nxt[k];
        if (r + wstride < p.R) {                                       // the next row's metadata loads under this row's work
#pragma unroll
            for (int k = 0; k < NR; ++k) nxt[k] = moe_row_meta(p, (size_t)e * p.Q + r + wstride + (size_t)k * p.R);
        }
        for (int g0 = 0; g0 < c; g0 += MOE_TOK) {
            const int nt = min(MOE_TOK, c - g0);
            float acc[NR][MOE_TOK];
#pragma unroll
            for (int k = 0; k < NR; ++k)
#pragma unroll
                for (int j = 0; j < MOE_TOK; ++j) acc[k][j] = 0.f;
            const bool fast = NR == 1 ? (m[0].nb <= 8 && (m[0].bit0 & 7) == 0)
                                      : (m[0].nb <= 8 && (m[0].bit0 & 7) == 0 && m[NR - 1].nb <= 8 && (m[NR - 1].bit0 & 7) == 0);
            constexpr int UN = 2;                                       // 256-column blocks whose ids are fetched together
            for (int col0 = lane * 8; col0 < p.P; col0 += 256 * UN) {
                uint64_t v[NR][UN];
                if (fast) {                                             // all the row bytes of this step in flight at once
#pragma unroll
                    for (int u = 0; u < UN; ++u)
#pragma unroll
                        for (int k = 0; k < NR; ++k) {
                            const int col = col0 + 256 * u;
                            v[k][u] = col < p.P ? load_8_fields(p.ids, (m[k].bit0 >> 3) + (int64_t)(col >> 3) * m[k].nb) : 0ull;
                        }
                }
#pragma unroll
                for (int u = 0; u < UN; ++u) {
                    const int col = col0 + 256 * u;
                    if (col >= p.P) break;
                    float wv[NR][8];
#pragma unroll
                    for (int k = 0; k < NR; ++k) {
                        if (fast) {
                            const uint32_t mask = (1u << m[k].nb) - 1u;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                wv[k][i] = __fmaf_rn(small_u2f((uint32_t)(v[k][u] >> (i * m[k].nb)) & mask), m[k].ts, m[k].ms);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                wv[k][i] = band(field_bytes(p.ids, m[k].bit0 + (int64_t)(col + i) * m[k].nb, m[k].nb), m[k].ts, m[k].ms);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < MOE_TOK; ++j) {
                        if (j < nt) {
                            const int pp = plist[g0 + j];
                            float x[8];
                            load_x8(p.X, (int64_t)(ACT == 2 ? pp : pp / p.topk) * p.P + col, x);
#pragma unroll
                            for (int k = 0; k < NR; ++k)
#pragma unroll
                                for (int i = 0; i < 8; ++i) acc[k][j] = __fmaf_rn(x[i], wv[k][i], acc[k][j]);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < MOE_TOK; ++j) {
                if (j < nt) {                                           // warp-uniform
#pragma unroll
                    for (int k = 0; k < NR; ++k)
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) acc[k][j] += __shfl_xor_sync(0xffffffffu, acc[k][j], o);
                    if (lane == 0) {
                        float v;
                        if (ACT == 0) {
                            const float gt = acc[0][j];
                            v = (gt / (1.0f + __expf(-gt))) * acc[NR - 1][j];
                        } else if (ACT == 1) {
                            const float u = fmaxf(acc[0][j], 0.f);
                            v = u * u;
                        } else {
                            v = acc[0][j];
                        }
                        p.out[(size_t)plist[g0 + j] * p.R + r] = v;
                    }
                }
            }
        }
    }
}

// out[t, d] = sum_j w[t, j] * Yd[t * topk + j, d], j ascending (qvb8_cuda.cu:936-947)
template <typename OutT>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float *__restrict__ Yd, const float *__restrict__ w,
                                                          OutT *__restrict__ out, int topk, int D, int M,
                                                          const int *__restrict__ valid) {
    const int t = blockIdx.y, d = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= M || d >= D) return;
    float a = 0.f;
    for (int j = 0; j < topk; ++j)                                      // a pair that was never computed counts as zero
        if (valid[t * topk + j]) a = __fmaf_rn(__ldg(w + t * topk + j), Yd[((size_t)t * topk + j) * D + d], a);
    out[(size_t)t * D + d] = narrow<OutT>(a);
}

struct MoeScratch {
    int64_t counts, lists, slots, nslots, bad, valid, Xf, H, Yd, total;
};
static MoeScratch moe_scratch(int64_t M, int64_t topk, int64_t E, int64_t Pup, int64_t R_up, int64_t Qdn) {
    MoeScratch s{};
    const int64_t npairs = M * topk;
    auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
    s.counts = 0;
    s.lists = s.counts + up(E * 4);
    s.slots = s.lists + up(E * M * 4);
    s.nslots = s.slots + up(E * 4);
    s.bad = s.nslots + 256;
    s.valid = s.bad + 256;
    s.Xf = s.valid + up(npairs * 4);
    s.H = s.Xf + up(M * Pup * 4);
    s.Yd = s.H + up(npairs * R_up * 4);
    s.total = s.Yd + up(npairs * Qdn * 4);
    return s;
}

static int check_stack(const qvb8_expert_stack *st, const char *who) {
    if (!st || !st->ids || !st->min_s || !st->tau_s || !st->nbits || !st->bit_off)
        return fail(QVB8_ERR_ARG, "%s: null expert stack", who);
    if (st->Q <= 0 || st->P <= 0 || st->Q > 0x7fffffff || st->P > 0x7fffffff || st->P % 8 != 0)
        return fail(QVB8_ERR_ARG, "%s: Q=%lld P=%lld (P must be a multiple of 8)", who, (long long)st->Q, (long long)st->P);
    if (!aligned(st->ids, 8)) return fail(QVB8_ERR_ALIGN, "%s: the stacked ids must be 8-byte aligned", who);
    return QVB8_OK;
}

}  // namespace qv

QV_API int64_t qvb8_moe_scratch_bytes(int64_t M, int64_t topk, int64_t E, int64_t Pup, int64_t Qup, int64_t Qdn, int act) {
    if (M <= 0 || topk <= 0 || E <= 0 || Pup <= 0 || Qup <= 0 || Qdn <= 0) return 0;
    return qv::moe_scratch(M, topk, E, Pup, act == 0 ? Qup / 2 : Qup, Qdn).total;
}

QV_API int qvb8_moe_experts(const void *X, int x_dtype, int64_t M, const int64_t *idx, const float *w, int64_t topk,
                            int64_t E, const qvb8_expert_stack *up, const qvb8_expert_stack *dn, int act, void *out,
                            void *scratch, int64_t scratch_bytes, void *stream) {
    using namespace qv;
    const char *who = act == 0 ? "qvb8_moe_experts" : "qvb8_moe_experts(relu2)";
    if (int rc = check_device(who)) return rc;
    if (int rc = check_stack(up, who)) return rc;
    if (int rc = check_stack(dn, who)) return rc;
    if (act != 0 && act != 1) return fail(QVB8_ERR_ARG, "%s: act must be 0 (gated SiLU) or 1 (relu^2)", who);
    if (!X || !idx || !w || !out) return fail(QVB8_ERR_ARG, "%s: null argument", who);
    if (x_dtype != QVB8_F16 && x_dtype != QVB8_BF16 && x_dtype != QVB8_F32) return fail(QVB8_ERR_ARG, "%s: bad X dtype", who);
    if (M <= 0 || topk <= 0 || E <= 0 || M * topk > 65535) return fail(QVB8_ERR_ARG, "%s: M=%lld topk=%lld E=%lld out of range", who, (long long)M, (long long)topk, (long long)E);
    const int64_t R_up = act == 0 ? up->Q / 2 : up->Q;
    if (act == 0 && up->Q % 2 != 0) return fail(QVB8_ERR_ARG, "%s: gate_up must have an even number of rows", who);
    if (R_up != dn->P) return fail(QVB8_ERR_ARG, "%s: up and down shapes disagree (%lld hidden vs %lld columns)", who, (long long)R_up, (long long)dn->P);
    if (!aligned(X, 16)) return fail(QVB8_ERR_ALIGN, "%s: X must be 16-byte aligned", who);
    const MoeScratch L = moe_scratch(M, topk, E, up->P, R_up, dn->Q);
    if (!scratch || scratch_bytes < L.total || !aligned(scratch, 256))
        return fail(QVB8_ERR_SCRATCH, "%s: scratch of %lld bytes (256-byte aligned) needed, %lld given", who, (long long)L.total, (long long)scratch_bytes);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    uint8_t *base = reinterpret_cast<uint8_t *>(scratch);
    MoeRoute route{reinterpret_cast<int *>(base + L.counts), reinterpret_cast<int *>(base + L.lists),
                   reinterpret_cast<int *>(base + L.slots), reinterpret_cast<int *>(base + L.nslots),
                   reinterpret_cast<int *>(base + L.bad), reinterpret_cast<int *>(base + L.valid)};
    const int npairs = (int)(M * topk);
    float *Xf = reinterpret_cast<float *>(base + L.Xf);
    const int64_t nx = M * up->P;
    moe_route_kernel<<<1 + (unsigned)((nx + 2047) / 2048), 256, 0, st>>>(idx, npairs, (int)E, (int)M, route, X, x_dtype, nx, Xf);
    if (int rc = cuda_status("qvb8_moe route")) return rc;
    const int max_slots = (int)(E < npairs ? E : npairs);
    float *H = reinterpret_cast<float *>(base + L.H), *Yd = reinterpret_cast<float *>(base + L.Yd);
    MoeRows a{Xf, (int)topk, up->ids, up->min_s, up->tau_s, up->nbits, up->bit_off, (int)up->Q, (int)up->P,
              (int)R_up, H, route, (int)M};
    // a few CTAs per expert, every warp walking several rows: short rows (a kilobyte or two) would otherwise be all
    // start-up latency
    auto row_blocks = [&](int64_t rows) {                              // about eight CTAs per SM over all experts
        const int64_t all = (rows + MOE_WARPS - 1) / MOE_WARPS, want = (1184 + max_slots - 1) / max_slots;
        return (unsigned)(all < want ? all : (want < 4 ? 4 : want));
    };
    const dim3 gu(row_blocks(R_up), (unsigned)max_slots);
    if (act == 0) moe_rows_kernel<0><<<gu, MOE_WARPS * 32, 0, st>>>(a);
    else moe_rows_kernel<1><<<gu, MOE_WARPS * 32, 0, st>>>(a);
    if (int rc = cuda_status("qvb8_moe up")) return rc;
    MoeRows b{H, (int)topk, dn->ids, dn->min_s, dn->tau_s, dn->nbits, dn->bit_off, (int)dn->Q, (int)dn->P,
              (int)dn->Q, Yd, route, (int)M};
    const dim3 gd(row_blocks(dn->Q), (unsigned)max_slots);
    moe_rows_kernel<2><<<gd, MOE_WARPS * 32, 0, st>>>(b);
    if (int rc = cuda_status("qvb8_moe down")) return rc;
    const dim3 gc((unsigned)((dn->Q + 255) / 256), (unsigned)M);
    if (x_dtype == QVB8_BF16)
        moe_combine_kernel<__nv_bfloat16><<<gc, 256, 0, st>>>(Yd, w, reinterpret_cast<__nv_bfloat16 *>(out), (int)topk, (int)dn->Q, (int)M, route.valid);
    else if (x_dtype == QVB8_F16)
        moe_combine_kernel<__half><<<gc, 256, 0, st>>>(Yd, w, reinterpret_cast<__half *>(out), (int)topk, (int)dn->Q, (int)M, route.valid);
    else
        moe_combine_kernel<float><<<gc, 256, 0, st>>>(Yd, w, reinterpret_cast<float *>(out), (int)topk, (int)dn->Q, (int)M, route.valid);
    return cuda_status("qvb8_moe combine");
}

// Expert index check of the last qvb8_moe_experts call that used `scratch` (after the stream has run it):
// 1 if a pair was left out (its expert index outside [0, E), or its token named one expert more than M times); such a
// pair contributes zero to the output.  Synchronises the host.
QV_API int qvb8_moe_bad_index(const void *scratch, int64_t M, int64_t topk, int64_t E, int64_t Pup, int64_t Qup, int64_t Qdn,
                              int act, int *bad) {
    using namespace qv;
    if (!scratch || !bad) return fail(QVB8_ERR_ARG, "qvb8_moe_bad_index: null argument");
    const MoeScratch L = moe_scratch(M, topk, E, Pup, act == 0 ? Qup / 2 : Qup, Qdn);
    if (cudaMemcpy(bad, reinterpret_cast<const uint8_t *>(scratch) + L.bad, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return cuda_status("qvb8_moe_bad_index");
    return QVB8_OK;
}
