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
//
// Up to 8 tokens with per-expert plans (qvb8_moe_plan_build): the STREAMING route.  Every selected expert becomes one
// job of the small-M streaming kernel (bulk-copy rings, tensor-core sums; qvb8_small_m.cu) with ALL tokens as its
// activations -- an m16n8k16 MMA has eight token columns whether one token chose the expert or all did -- so the job
// list depends on the routing only through WHICH experts it names.  The route kernel writes the two job tables (up,
// down) into device memory and the streaming kernel reads them from there:
//   route + job tables -> up jobs (U[slot] = X W_up^T) -> activation (H[slot], per-row power-of-two scaling)
//   -> down jobs (Yd[slot] = H W_dn^T) -> combine (out[t] = sum_j w[t,j] * Yd[slot(e_tj)][t] * 2^k).
// The hidden activations pass through the streaming kernel's fp16 staging; each (slot, token) row is first scaled by
// the power of two that puts its largest magnitude in [2^14, 2^15), so nothing saturates or goes subnormal, and the
// scale is undone exactly in the combine step (relative error of a hidden value <= 2^-11, far inside the 1e-2 bound).
#include "common.cuh"
#include "plan.cuh"

namespace qv {

constexpr int MOE_WARPS = 8;
constexpr int MOE_STREAM_TOKENS = 8;       // the streaming route's token limit (one MMA token group)
constexpr int MOE_STREAM_SLOTS = 128;      // ... and its limit on distinct experts per call
constexpr int MOE_TOK = 4;                 // tokens per pass over a row

struct MoeJobs {                           // what the route kernel needs to write the streaming route's job tables
    JobDesc *up, *dn;                      // [cap] tables, null: no tables wanted
    int *slot_of;                          // [E] slot of expert e, -1 if not chosen
    const uint8_t *up_ids, *dn_ids;
    const uint8_t *up_nbits, *dn_nbits;
    const int64_t *up_bitoff, *dn_bitoff;
    const uint8_t *up_plan, *dn_plan;      // per expert: a plan (plan_layout(Q, 0)), `*_stride` bytes apart
    int64_t up_stride, dn_stride, up_tiles_off, dn_tiles_off;
    int up_Q, up_P, dn_Q, dn_P, up_ntiles, dn_ntiles, up_units, dn_units;
    const void *X;                         // (M, up_P) activations as given
    int x_dtype;
    float *U, *H, *Yd;                     // [cap][M][up_Q], [cap][M][dn_P], [cap][M][dn_Q]
};

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
                                                        float *__restrict__ Xf, const MoeJobs jb) {
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
    __shared__ int s_cnt[1024];                                         // counts of the first 1024 experts
    __shared__ int s_idx[2048];                                         // the pairs' experts (-1: out of range), when they fit
    const bool in_smem = npairs <= 2048;
    if (threadIdx.x == 0) any_bad = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < npairs; p += blockDim.x) {
        const int64_t e = idx[p];
        const bool ok = e >= 0 && e < E;
        if (!ok) any_bad = 1;
        if (in_smem) s_idx[p] = ok ? (int)e : -1;
        r.valid[p] = 0;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int p = 0; p < npairs; ++p)
            if (in_smem ? s_idx[p] == e : idx[p] == e) {
                if (c < M) { r.lists[(size_t)e * M + c++] = p; r.valid[p] = 1; }
                else any_bad = 1;
            }
        r.counts[e] = c;
        if (e < 1024) s_cnt[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int n = 0;
        for (int e = 0; e < E; ++e)
            if ((e < 1024 ? s_cnt[e] : r.counts[e]) > 0) r.slots[n++] = e;
        *r.nslots = n;
        *r.bad = any_bad;
    }
    if (jb.up == nullptr) return;
    // the streaming route: one up job and one down job per distinct expert, slot order = expert order
    __syncthreads();
    const int n = *r.nslots;
    for (int e = threadIdx.x; e < E; e += blockDim.x) jb.slot_of[e] = -1;
    __syncthreads();
    for (int s = threadIdx.x; s < n; s += blockDim.x) {
        const int e = r.slots[s];
        jb.slot_of[e] = s;
        JobDesc u{};
        u.ids = jb.up_ids; u.nbits = jb.up_nbits + (size_t)e * jb.up_Q; u.bit_off = jb.up_bitoff + (size_t)e * jb.up_Q;
        u.tiles = reinterpret_cast<const TileDesc *>(jb.up_plan + (size_t)e * jb.up_stride + jb.up_tiles_off);
        u.esc_ent = nullptr;
        u.X = jb.X; u.Y = jb.U + (size_t)s * M * jb.up_Q;
        u.ntiles = jb.up_ntiles; u.Q = jb.up_Q; u.P = jb.up_P; u.nc_total = jb.up_P / 128;
        u.x_dtype = jb.x_dtype; u.x_mode = 0; u.unit0 = s * jb.up_units; u.yflags = 0; u.kc0 = 0; u.nsk_part = 0;
        jb.up[s] = u;
        JobDesc d{};
        d.ids = jb.dn_ids; d.nbits = jb.dn_nbits + (size_t)e * jb.dn_Q; d.bit_off = jb.dn_bitoff + (size_t)e * jb.dn_Q;
        d.tiles = reinterpret_cast<const TileDesc *>(jb.dn_plan + (size_t)e * jb.dn_stride + jb.dn_tiles_off);
        d.esc_ent = nullptr;
        d.X = jb.H + (size_t)s * M * jb.dn_P; d.Y = jb.Yd + (size_t)s * M * jb.dn_Q;
        d.ntiles = jb.dn_ntiles; d.Q = jb.dn_Q; d.P = jb.dn_P; d.nc_total = jb.dn_P / 128;
        d.x_dtype = QVB8_F32; d.x_mode = 0; d.unit0 = s * jb.dn_units; d.yflags = 0; d.kc0 = 0; d.nsk_part = 0;
        jb.dn[s] = d;
    }
}

// Streaming route, between the up and the down jobs: block (slot, token) turns row U[slot][t] into the hidden row
// H[slot][t] = act(U) * 2^-k, k chosen so that the row's largest magnitude lies in [2^14, 2^15) (k = 0 for a zero row);
// kexp[slot][t] = k.  ACT 0: U holds gate (first I values) and up (next I); ACT 1: relu^2 of the I values.
template <int ACT>
__global__ void __launch_bounds__(256) moe_hidden_kernel(const float *__restrict__ U, float *__restrict__ H,
                                                         int *__restrict__ kexp, const int *__restrict__ nslots, int M, int I) {
    const int s = blockIdx.x, t = blockIdx.y;
    if (s >= *nslots) return;
    const int QU = ACT == 0 ? 2 * I : I;
    const float *u = U + ((size_t)s * M + t) * QU;
    float *h = H + ((size_t)s * M + t) * I;
    auto value = [&](int i) {
        if (ACT == 0) {
            const float g = u[i];
            return (g / (1.0f + __expf(-g))) * u[I + i];
        }
        const float v = fmaxf(u[i], 0.f);
        return v * v;
    };
    float amax = 0.f;
    for (int i = threadIdx.x; i < I; i += blockDim.x) {
        const float v = fabsf(value(i));
        if (v < 3.0e38f) amax = fmaxf(amax, v);                        // (infinities and NaNs keep their own scale-free fate)
    }
    __shared__ float red[8];
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
    for (int k = 1; k < 8; ++k) amax = fmaxf(amax, red[k]);
    int k = 0;
    if (amax > 0.f) {
        int e;
        frexpf(amax, &e);                                               // amax = m * 2^e, m in [0.5, 1)
        k = e - 15;                                                     // amax * 2^-k in [2^14, 2^15)
    }
    if (threadIdx.x == 0) kexp[s * M + t] = k;
    for (int i = threadIdx.x; i < I; i += blockDim.x) h[i] = ldexpf(value(i), -k);
}

// Streaming route: out[t, d] = sum_j w[t, j] * Yd[slot(e_tj)][t][d] * 2^k[slot][t], j ascending; invalid pairs count zero
template <typename OutT>
__global__ void __launch_bounds__(256) moe_combine_slots_kernel(const float *__restrict__ Yd, const float *__restrict__ w,
                                                                const int64_t *__restrict__ idx, const int *__restrict__ slot_of,
                                                                const int *__restrict__ kexp, OutT *__restrict__ out, int topk,
                                                                int D, int M, int E, const int *__restrict__ valid) {
    const int t = blockIdx.y, d = blockIdx.x * blockDim.x + threadIdx.x;
    // the token's pairs once per block: slot (-1 = the pair counts zero), routing weight, scale exponent
    constexpr int TOPK_SMEM = 64;
    __shared__ int s_slot[TOPK_SMEM], s_k[TOPK_SMEM];
    __shared__ float s_w[TOPK_SMEM];
    const bool staged = topk <= TOPK_SMEM;
    if (staged && t < M) {
        for (int j = threadIdx.x; j < topk; j += blockDim.x) {
            const int sl = valid[t * topk + j] ? slot_of[(int)idx[t * topk + j]] : -1;
            s_slot[j] = sl;
            s_w[j] = w[t * topk + j];
            s_k[j] = sl >= 0 ? kexp[sl * M + t] : 0;
        }
    }
    __syncthreads();
    if (t >= M || d >= D) return;
    float a = 0.f;
    for (int j = 0; j < topk; ++j) {
        int sl, k;
        float wj;
        if (staged) { sl = s_slot[j]; k = s_k[j]; wj = s_w[j]; }
        else {
            sl = valid[t * topk + j] ? slot_of[(int)idx[t * topk + j]] : -1;
            k = sl >= 0 ? kexp[sl * M + t] : 0;
            wj = w[t * topk + j];
        }
        if (sl >= 0) a = __fmaf_rn(wj, ldexpf(Yd[((size_t)sl * M + t) * D + d], k), a);
    }
    out[(size_t)t * D + d] = narrow<OutT>(a);
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
    // the streaming route's sections (present when M <= MOE_STREAM_TOKENS), after the others
    int64_t slot_of, kexp, jobs_up, jobs_dn, U, Hs, Yds;
    int cap;                                                           // slots the route can produce
};
static MoeScratch moe_scratch(int64_t M, int64_t topk, int64_t E, int64_t Pup, int64_t R_up, int64_t Qdn, int64_t Qup_rows) {
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
    s.cap = (int)(E < npairs ? E : npairs);
    if (M <= MOE_STREAM_TOKENS && s.cap <= MOE_STREAM_SLOTS) {
        const int64_t Qup = Qup_rows;
        s.slot_of = s.total;
        s.kexp = s.slot_of + up(E * 4);
        s.jobs_up = s.kexp + up((int64_t)s.cap * M * 4);
        s.jobs_dn = s.jobs_up + up((int64_t)s.cap * (int64_t)sizeof(JobDesc));
        s.U = s.jobs_dn + up((int64_t)s.cap * (int64_t)sizeof(JobDesc));
        s.Hs = s.U + up((int64_t)s.cap * M * Qup * 4);
        s.Yds = s.Hs + up((int64_t)s.cap * M * R_up * 4);
        s.total = s.Yds + up((int64_t)s.cap * M * Qdn * 4);
    }
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
    return qv::moe_scratch(M, topk, E, Pup, act == 0 ? Qup / 2 : Qup, Qdn, Qup).total;
}

/* Bytes of the plans of all E experts of a stack with Q rows per expert (one plan per expert, back to back). */
QV_API int64_t qvb8_moe_plan_bytes(int64_t E, int64_t Q) {
    if (E <= 0 || Q <= 0) return 0;
    return E * qv::plan_layout(Q, 0).total;
}

/* Builds the per-expert plans of a stack (the row ordering of qvb8_plan_build, once per expert) into `plan`. */
QV_API int qvb8_moe_plan_build(const qvb8_expert_stack *stk, int64_t E, void *plan, int64_t plan_bytes, void *stream) {
    using namespace qv;
    if (int rc = check_device("qvb8_moe_plan_build")) return rc;
    if (int rc = check_stack(stk, "qvb8_moe_plan_build")) return rc;
    const int64_t need = qvb8_moe_plan_bytes(E, stk->Q);
    if (E <= 0 || !plan || plan_bytes < need || !aligned(plan, 256))
        return fail(QVB8_ERR_SCRATCH, "qvb8_moe_plan_build: plan buffer of %lld bytes (256-byte aligned) needed", (long long)need);
    const int64_t stride = plan_layout(stk->Q, 0).total;
    for (int64_t e = 0; e < E; ++e) {
        qvb8_pack w{};
        w.ids = stk->ids; w.ids_bytes = stk->ids_bytes;
        w.min_s = stk->min_s + e * stk->Q; w.tau_s = stk->tau_s + e * stk->Q;
        w.nbits = stk->nbits + e * stk->Q; w.bit_off = stk->bit_off + e * stk->Q;
        w.Q = stk->Q; w.P = stk->P; w.esc_idx = nullptr; w.esc_vals = nullptr; w.n_esc = 0;
        if (int rc = qvb8_plan_build(&w, reinterpret_cast<uint8_t *>(plan) + e * stride, stride, stream)) return rc;
    }
    return QVB8_OK;
}

/* 1 when qvb8_moe_experts_planned, given plans, runs this shape through the streaming kernel; 0 when it takes the
 * plan-less route (too many tokens or distinct experts, column counts that are no multiples of 128, unaligned stacks). */
QV_API int qvb8_moe_streams(int64_t M, int64_t topk, int64_t E, const qvb8_expert_stack *up, const qvb8_expert_stack *dn) {
    using namespace qv;
    if (!up || !dn || M <= 0 || topk <= 0 || E <= 0) return 0;
    const MoeScratch L = moe_scratch(M, topk, E, up->P, dn->P, dn->Q, up->Q);
    if (!L.Yds || !aligned(up->ids, 16) || !aligned(dn->ids, 16)) return 0;
    return small_m_devlist_units(M, up->P, L.cap, plan_layout(up->Q, 0).max_tiles) > 0 &&
           small_m_devlist_units(M, dn->P, L.cap, plan_layout(dn->Q, 0).max_tiles) > 0;
}

QV_API int qvb8_moe_experts_planned(const void *X, int x_dtype, int64_t M, const int64_t *idx, const float *w, int64_t topk,
                                    int64_t E, const qvb8_expert_stack *up, const qvb8_expert_stack *dn, const void *up_plan,
                                    const void *dn_plan, int act, void *out, void *scratch, int64_t scratch_bytes,
                                    void *stream) {
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
    const MoeScratch L = moe_scratch(M, topk, E, up->P, R_up, dn->Q, up->Q);
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
    // ---- the streaming route: every distinct expert one job of the small-M streaming kernel, all tokens as activations
    const PlanLayout pu = plan_layout(up->Q, 0), pd = plan_layout(dn->Q, 0);
    const int units_up = (up_plan && dn_plan && L.Yds) ? small_m_devlist_units(M, up->P, L.cap, pu.max_tiles) : 0;
    const int units_dn = units_up ? small_m_devlist_units(M, dn->P, L.cap, pd.max_tiles) : 0;
    if (units_up > 0 && units_dn > 0 && aligned(up->ids, 16) && aligned(dn->ids, 16) && aligned(up_plan, 256) &&
        aligned(dn_plan, 256)) {
        MoeJobs jb{};
        jb.up = reinterpret_cast<JobDesc *>(base + L.jobs_up);
        jb.dn = reinterpret_cast<JobDesc *>(base + L.jobs_dn);
        jb.slot_of = reinterpret_cast<int *>(base + L.slot_of);
        jb.up_ids = up->ids; jb.dn_ids = dn->ids; jb.up_nbits = up->nbits; jb.dn_nbits = dn->nbits;
        jb.up_bitoff = up->bit_off; jb.dn_bitoff = dn->bit_off;
        jb.up_plan = reinterpret_cast<const uint8_t *>(up_plan); jb.dn_plan = reinterpret_cast<const uint8_t *>(dn_plan);
        jb.up_stride = pu.total; jb.dn_stride = pd.total; jb.up_tiles_off = pu.tiles; jb.dn_tiles_off = pd.tiles;
        jb.up_Q = (int)up->Q; jb.up_P = (int)up->P; jb.dn_Q = (int)dn->Q; jb.dn_P = (int)dn->P;
        jb.up_ntiles = pu.max_tiles; jb.dn_ntiles = pd.max_tiles; jb.up_units = units_up; jb.dn_units = units_dn;
        jb.X = X; jb.x_dtype = x_dtype;
        jb.U = reinterpret_cast<float *>(base + L.U);
        jb.H = reinterpret_cast<float *>(base + L.Hs);
        jb.Yd = reinterpret_cast<float *>(base + L.Yds);
        int *kexp = reinterpret_cast<int *>(base + L.kexp);
        moe_route_kernel<<<1, 256, 0, st>>>(idx, npairs, (int)E, (int)M, route, X, x_dtype, 0, Xf, jb);
        if (int rc = cuda_status("qvb8_moe route")) return rc;
        if (int rc = small_m_devlist_launch(jb.up, route.nslots, L.cap, M, up->P, pu.max_tiles, false, st)) return rc;
        const dim3 gh((unsigned)L.cap, (unsigned)M);
        if (act == 0) moe_hidden_kernel<0><<<gh, 256, 0, st>>>(jb.U, jb.H, kexp, route.nslots, (int)M, (int)R_up);
        else moe_hidden_kernel<1><<<gh, 256, 0, st>>>(jb.U, jb.H, kexp, route.nslots, (int)M, (int)R_up);
        if (int rc = cuda_status("qvb8_moe hidden")) return rc;
        if (int rc = small_m_devlist_launch(jb.dn, route.nslots, L.cap, M, dn->P, pd.max_tiles, false, st)) return rc;
        const dim3 gs((unsigned)((dn->Q + 255) / 256), (unsigned)M);
        if (x_dtype == QVB8_BF16)
            moe_combine_slots_kernel<__nv_bfloat16><<<gs, 256, 0, st>>>(jb.Yd, w, idx, jb.slot_of, kexp, reinterpret_cast<__nv_bfloat16 *>(out), (int)topk, (int)dn->Q, (int)M, (int)E, route.valid);
        else if (x_dtype == QVB8_F16)
            moe_combine_slots_kernel<__half><<<gs, 256, 0, st>>>(jb.Yd, w, idx, jb.slot_of, kexp, reinterpret_cast<__half *>(out), (int)topk, (int)dn->Q, (int)M, (int)E, route.valid);
        else
            moe_combine_slots_kernel<float><<<gs, 256, 0, st>>>(jb.Yd, w, idx, jb.slot_of, kexp, reinterpret_cast<float *>(out), (int)topk, (int)dn->Q, (int)M, (int)E, route.valid);
        return cuda_status("qvb8_moe combine");
    }
    moe_route_kernel<<<1 + (unsigned)((nx + 2047) / 2048), 256, 0, st>>>(idx, npairs, (int)E, (int)M, route, X, x_dtype, nx, Xf, MoeJobs{});
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

QV_API int qvb8_moe_experts(const void *X, int x_dtype, int64_t M, const int64_t *idx, const float *w, int64_t topk,
                            int64_t E, const qvb8_expert_stack *up, const qvb8_expert_stack *dn, int act, void *out,
                            void *scratch, int64_t scratch_bytes, void *stream) {
    return qvb8_moe_experts_planned(X, x_dtype, M, idx, w, topk, E, up, dn, nullptr, nullptr, act, out, scratch,
                                    scratch_bytes, stream);
}

// Expert index check of the last qvb8_moe_experts call that used `scratch` (after the stream has run it):
// 1 if a pair was left out (its expert index outside [0, E), or its token named one expert more than M times); such a
// pair contributes zero to the output.  Synchronises the host.
QV_API int qvb8_moe_bad_index(const void *scratch, int64_t M, int64_t topk, int64_t E, int64_t Pup, int64_t Qup, int64_t Qdn,
                              int act, int *bad) {
    using namespace qv;
    if (!scratch || !bad) return fail(QVB8_ERR_ARG, "qvb8_moe_bad_index: null argument");
    const MoeScratch L = moe_scratch(M, topk, E, Pup, act == 0 ? Qup / 2 : Qup, Qdn, Qup);
    if (cudaMemcpy(bad, reinterpret_cast<const uint8_t *>(scratch) + L.bad, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return cuda_status("qvb8_moe_bad_index");
    return QVB8_OK;
}
