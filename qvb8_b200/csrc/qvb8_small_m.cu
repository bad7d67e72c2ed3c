// QVB8 small-M fused decode-in-matmul for sm_100a:  Y[m, q] = sum_c X[m, c] * W[q, c],  1 <= M <= 48,
// W read ONCE from HBM as bit-packed ids and never materialised.
//
// Replaces the reference's GEMV family and its mma.sync verify kernel
// (formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:306-453 qvb8_gemv_multi_v3, :463-489 split-K, :1813-2441 qvb8_mma_*).
//
// Arithmetic.  With w = min_s + id * tau_s the row sum factors (the identity the reference states at
// qvb8_cuda.cu:3-9):   y[m, q] = min_s[q] * sum_c x[m, c]  +  tau_s[q] * sum_c x[m, c] * id[q, c].
// The ids are small integers, exact in fp16, so the inner sum runs on the tensor cores (fp16 x fp16 -> fp32,
// products exact, fp32 accumulation) and the per-weight CUDA-core work is only the bit extraction.  The weight
// is therefore the un-narrowed band value, the contract of the reference's M <= 8 GEMV; X is narrowed to saturated
// fp16 first, as every fp16-mode path of the reference does (:761-841).
//
// Roofline: HBM.  Per weight the kernel moves nbits/8 bytes (about 0.8) and spends ~1.5 issue slots; the stream is
// staged through shared memory with 16-byte cp.async copies (each warp keeps NST row-chunks in flight), so the
// load pattern seen by HBM is whole 16-byte-aligned row segments while the fragment reads happen in shared memory.
//
// Work split.  A CTA owns 128 consecutive output rows and one K-range.  Rows of a pack have different widths, so the
// CTA first sorts its rows by width into 16-row tiles of ONE width (shared-memory lists; no precomputed ordering is
// needed).  A warp takes a tile, and for every 128-column chunk: thread (g = lane / 4, t = lane % 4) owns the 32 ids
// of rows g and g + 8 that start at column 32 t -- exactly nb 32-bit words -- and turns them into the A fragments of
// eight m16n8k16 MMAs.  Two ids are converted per instruction: a funnel shift puts one id in the low half-word
// and one in the high half-word of a register, `(r & mask) | 0x64006400` makes the two fp16 numbers 1024 + id * 2^e,
// and one HFMA2 removes the 1024 and the 2^e exactly.  The B fragments are the activations, staged once per CTA as
// fp16 in the order the fragments want.  K-ranges of one row block are summed in a fixed order by the last CTA of
// the block to finish (a ticket counter), so results are identical from run to run.
#include "common.cuh"

namespace qv {

int launch_fix_escapes(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y, cudaStream_t st);
int launch_small_m_generic(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y,
                           cudaStream_t st);
int check_small_m_args(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, const float *Y,
                       const char *who);

constexpr int RB = 128;             // output rows per CTA
constexpr int NWARP = 8;            // warps per CTA
constexpr int KC = 128;             // columns per chunk (one cp.async stage of a tile)
constexpr int NST = 4;              // stages in flight per warp
constexpr int STAGE_BYTES = 16 * 144;   // 16 rows x (16 * nb bytes, +16 pad for nb = 8)
constexpr int MAXTILES = 16;        // 128 rows in <= 7 width classes make at most 8 + 6 tiles
constexpr int NCLASS = 7;           // widths 3..8 -> class 0..5; every other width -> class 6 (per-element path)
constexpr int XS_MAX_BYTES = 64 * 1024;
constexpr int64_t TICKET_BYTES = 64 * 1024;   // fixed-size counter area at the START of the scratch, so that calls of
                                              // different sizes sharing one scratch never find partial sums in it
constexpr int MAX_TICKET_BLOCKS = (int)(TICKET_BYTES / 4);

struct TileTable {
    int ntiles;
    int tile_nb[MAXTILES];          // width of the tile's rows; 0 = per-element class
    int tile_cnt[MAXTILES];         // real rows in the tile (the rest is padding)
    int row[MAXTILES][16];          // global row index, -1 = padding
    uint32_t base16[MAXTILES][16];  // byte offset of the row in `ids`, in 16-byte units
    float ms[MAXTILES][16];
    float ts[MAXTILES][16];
    int list[NCLASS][RB];           // scratch of the classification: local row numbers per class
    int count[NCLASS];
    float sumx[48];
    int is_last;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Pairing of a width: ids f and f + D share a register; the low one sits at mantissa bit E, the high one at bit 0
// of the upper half-word (nb * D == 16 - E).
template <int NB> struct Pairing;
template <> struct Pairing<8> { static constexpr int D = 2, E = 0; };
template <> struct Pairing<7> { static constexpr int D = 2, E = 2; };
template <> struct Pairing<6> { static constexpr int D = 2, E = 4; };
template <> struct Pairing<5> { static constexpr int D = 4, E = -4; };   // high id shifted instead: see pair_reg
template <> struct Pairing<4> { static constexpr int D = 4, E = 0; };
template <> struct Pairing<3> { static constexpr int D = 4, E = 4; };

// Register holding fp16(id[fa]) in the low half and fp16(id[fa + D]) in the high half, from the nb words W of a
// thread's 32-id block.  E >= 0: low id at mantissa bit E, high id at bit 0.  E < 0: low id at bit 0, high id at
// mantissa bit -E.  All shifts and masks fold to constants after unrolling.
template <int NB>
__device__ __forceinline__ uint32_t pair_reg(const uint32_t (&W)[NB], int fa) {
    constexpr int D = Pairing<NB>::D, E = Pairing<NB>::E;
    constexpr int EL = E > 0 ? E : 0;            // mantissa shift of the low id
    constexpr int EH = E < 0 ? -E : 0;           // mantissa shift of the high id
    static_assert(NB * D == 16 + EH - EL, "pairing does not line the two ids up");
    static_assert(EL + NB <= 10 && EH + NB <= 10, "id does not fit the fp16 mantissa");
    constexpr uint32_t FM = (1u << NB) - 1u;
    constexpr uint32_t MASK = (FM << EL) | (FM << (16 + EH));
    const int s = NB * fa - EL;                  // bit of the block that must land on bit 0
    uint32_t r;
    if (s < 0) {
        r = W[0] << (-s);
    } else {
        const int wi = s >> 5, sh = s & 31;
        const int top = sh + 16 + EH + NB;       // one past the highest bit needed, relative to W[wi]
        if (sh == 0) r = W[wi];
        else if (top <= 32) r = W[wi] >> sh;
        else r = __funnelshift_r(W[wi], W[wi + 1 < NB ? wi + 1 : wi], sh);
    }
    r = (r & MASK) | 0x64006400u;                // two fp16 numbers 1024 + id * 2^shift
    const float sl = 1.0f / (float)(1 << EL), shh = 1.0f / (float)(1 << EH);
    const __half2 scale = __floats2half2_rn(sl, shh);
    const __half2 bias = __floats2half2_rn(-1024.0f * sl, -1024.0f * shh);
    const __half2 v = __hfma2(*reinterpret_cast<const __half2 *>(&r), scale, bias);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// The nb words of a thread's block, with the widest conflict-free shared-memory loads for that width.
template <int NB>
__device__ __forceinline__ void load_block(uint32_t addr, uint32_t (&W)[NB]) {
    if constexpr (NB == 8) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(W[0]), "=r"(W[1]), "=r"(W[2]), "=r"(W[3]) : "r"(addr));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(W[4]), "=r"(W[5]), "=r"(W[6]), "=r"(W[7]) : "r"(addr + 16));
    } else if constexpr (NB == 4) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(W[0]), "=r"(W[1]), "=r"(W[2]), "=r"(W[3]) : "r"(addr));
    } else if constexpr (NB == 6) {
#pragma unroll
        for (int k = 0; k < 6; k += 2)
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(W[k]), "=r"(W[k + 1]) : "r"(addr + 4 * k));
    } else {
#pragma unroll
        for (int k = 0; k < NB; ++k) asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(W[k]) : "r"(addr + 4 * k));
    }
}

__device__ __forceinline__ int row_stride(int nb) { return nb == 8 ? 144 : 16 * nb; }

// One 128-column chunk of a 16-row tile of width NB: 8 MMAs per token group.
template <int NB, int NT>
__device__ __forceinline__ void chunk_mma(uint32_t stage, uint32_t xs_chunk, int MP, int lane, float (&acc)[NT][4]) {
    constexpr int D = Pairing<NB>::D;
    const int g = lane >> 2, t = lane & 3;
    const int RS = NB == 8 ? 144 : 16 * NB;
    uint32_t Wa[NB], Wb[NB];
    load_block<NB>(stage + g * RS + t * 4 * NB, Wa);
    load_block<NB>(stage + (g + 8) * RS + t * 4 * NB, Wb);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // activations of columns 32 t + 8 i .. + 7 for this thread's token(s): one 16-byte slot per token
        uint32_t xw[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int m = 8 * n + g;
            xw[n][0] = xw[n][1] = xw[n][2] = xw[n][3] = 0u;
            if (m < MP) {
                const uint32_t a = xs_chunk + (uint32_t)(((i * 4 + t) * MP + m) * 16);
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(xw[n][0]), "=r"(xw[n][1]), "=r"(xw[n][2]), "=r"(xw[n][3]) : "r"(a));
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // ids of this MMA: D == 2 -> {8i+4h .. 8i+4h+3} paired (f, f+2);  D == 4 -> {8i+2h, +1, +4, +5} paired (f, f+4)
            const int f0 = D == 2 ? 8 * i + 4 * h : 8 * i + 2 * h;
            const uint32_t a0 = pair_reg<NB>(Wa, f0), a2 = pair_reg<NB>(Wa, f0 + 1);
            const uint32_t a1 = pair_reg<NB>(Wb, f0), a3 = pair_reg<NB>(Wb, f0 + 1);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                uint32_t lo, hi;                   // the two words holding x[f0 - 8i], x[f0 + 1 - 8i] and their partners
                if (D == 2) { lo = xw[n][2 * h]; hi = xw[n][2 * h + 1]; }
                else        { lo = xw[n][h];     hi = xw[n][h + 2]; }
                const uint32_t b0 = __byte_perm(lo, hi, 0x5410), b1 = __byte_perm(lo, hi, 0x7632);
                mma16816(acc[n], a0, a1, a2, a3, b0, b1);
            }
        }
    }
}

// Position (in halves) of X[m, c] inside the staged activation array; c is relative to the CTA's first column.
__device__ __forceinline__ int xs_index(int c, int m, int MP) {
    const int chunk = c >> 7, t = (c >> 5) & 3, i = (c >> 3) & 3, e = c & 7;
    return ((((chunk * 4 + i) * 4 + t) * MP + m) << 3) + e;
}

template <int XT>
__device__ __forceinline__ void stage_x8(const void *__restrict__ X, int64_t off, __half (&h)[8]) {
    if constexpr (XT == QVB8_F16) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(X) + off));
        const __half2 *p = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
        for (int k = 0; k < 4; ++k) { h[2 * k] = __low2half(p[k]); h[2 * k + 1] = __high2half(p[k]); }
    } else if constexpr (XT == QVB8_BF16) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(X) + off));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            h[2 * k] = sat_half(__uint_as_float(w[k] << 16));
            h[2 * k + 1] = sat_half(__uint_as_float(w[k] & 0xffff0000u));
        }
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(X) + off));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(X) + off) + 1);
        h[0] = sat_half(a.x); h[1] = sat_half(a.y); h[2] = sat_half(a.z); h[3] = sat_half(a.w);
        h[4] = sat_half(b.x); h[5] = sat_half(b.y); h[6] = sat_half(b.z); h[7] = sat_half(b.w);
    }
}

struct SmallMParams {
    const uint8_t *ids;
    const float *min_s;
    const float *tau_s;
    const uint8_t *nbits;
    const int64_t *bit_off;
    const void *X;
    float *Y;          // (M, Q)
    float *part;       // (S, M, Q) partial sums when S > 1
    int *ticket;       // one counter per row block when S > 1 (zero on entry, zero on exit)
    int Q, P, M, MP;   // MP: token slots per column group in shared memory (>= M)
    int S;             // K-ranges
    int nc_per;        // chunks per K-range (the last range may be shorter)
    int nc_total;      // P / 128
};

template <int XT, int NT>
__global__ void __launch_bounds__(NWARP * 32, 2) small_m_kernel(const SmallMParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ TileTable tt;
    uint8_t *ring = smem;                                              // NWARP * NST * STAGE_BYTES
    __half *xs = reinterpret_cast<__half *>(smem + NWARP * NST * STAGE_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = blockIdx.x * RB;
    const int nrows = min(RB, p.Q - q0);
    const int split = blockIdx.y;
    const int kc0 = split * p.nc_per;                                  // first chunk of this K-range
    const int NC = min(p.nc_per, p.nc_total - kc0);                    // chunks in this K-range (>= 1 by construction)

    // ---- 1. sort the block's rows by width into tiles (warp 0; stable, so the order is the same on every run)
    if (warp == 0) {
        int cnt[NCLASS];
#pragma unroll
        for (int c = 0; c < NCLASS; ++c) cnt[c] = 0;
        for (int r0 = 0; r0 < RB; r0 += 32) {
            const int r = r0 + lane;
            int cls = -1;
            if (r < nrows) {
                const int nb = __ldg(p.nbits + q0 + r);
                const bool byte16 = (__ldg(p.bit_off + q0 + r) & 127) == 0;      // row starts on a 16-byte boundary
                cls = (nb >= 3 && nb <= 8 && byte16) ? nb - 3 : NCLASS - 1;
            }
#pragma unroll
            for (int c = 0; c < NCLASS; ++c) {
                const uint32_t mk = __ballot_sync(0xffffffffu, cls == c);
                if (cls == c) tt.list[c][cnt[c] + __popc(mk & ((1u << lane) - 1u))] = r;
                cnt[c] += __popc(mk);
            }
        }
        __syncwarp();
        int nt = 0;
#pragma unroll
        for (int c = 0; c < NCLASS; ++c) {
            for (int i0 = 0; i0 < cnt[c]; i0 += 16) {
                if (lane < 16) {
                    const int i = i0 + lane;
                    int row = -1; uint32_t b16 = 0; float ms = 0.f, ts = 0.f;
                    if (i < cnt[c]) {
                        row = q0 + tt.list[c][i];
                        b16 = (uint32_t)(__ldg(p.bit_off + row) >> 7);
                        ms = __ldg(p.min_s + row); ts = __ldg(p.tau_s + row);
                    }
                    tt.row[nt][lane] = row; tt.base16[nt][lane] = b16; tt.ms[nt][lane] = ms; tt.ts[nt][lane] = ts;
                }
                if (lane == 0) { tt.tile_nb[nt] = c == NCLASS - 1 ? 0 : c + 3; tt.tile_cnt[nt] = min(16, cnt[c] - i0); }
                ++nt;
            }
        }
        if (lane == 0) tt.ntiles = nt;
    }
    __syncthreads();

    // ---- 2. per-warp unit list (tile, chunk) and the first NST - 1 copies (weights do not depend on X)
    const int ntiles = tt.ntiles;
    const int n_my = warp < ntiles ? (ntiles - warp + NWARP - 1) / NWARP : 0;
    const int units = n_my * NC;
    const uint32_t ring_w = smem_u32(ring + warp * NST * STAGE_BYTES);
    auto issue = [&](int u) {
        const int tile = warp + (u / NC) * NWARP, chunk = u - (u / NC) * NC;
        const int nb = tt.tile_nb[tile];
        if (nb == 0) return;                                            // per-element class reads global memory itself
        const int pieces = tt.tile_cnt[tile] * nb;                      // 16-byte pieces of this row-chunk set
        const uint32_t magic = (65536u + nb - 1) / nb;
        const int RS = row_stride(nb);
        const uint32_t dst0 = ring_w + (u % NST) * STAGE_BYTES;
        for (int pc = lane; pc < pieces; pc += 32) {
            const int r = (int)((pc * magic) >> 16), j = pc - r * nb;
            const uint8_t *src = p.ids + ((int64_t)tt.base16[tile][r] + (int64_t)(kc0 + chunk) * nb + j) * 16;
            cp_async16(dst0 + r * RS + j * 16, src);
        }
    };
#pragma unroll
    for (int u = 0; u < NST - 1; ++u) {
        if (u < units) issue(u);
        cp_async_commit();
    }

    // ---- 3. stage the activations of this K-range as fp16 in fragment order; per-token sums
    {
        const int MP = p.MP, groups = NC * 16;                          // 8-column groups in the range
        const int64_t col0 = (int64_t)kc0 * KC;
        for (int idx = tid; idx < MP * groups; idx += NWARP * 32) {
            const int m = idx / groups, u8 = idx - m * groups;         // u8: natural 8-column group number
            __half h[8];
            if (m < p.M) {
                stage_x8<XT>(p.X, (int64_t)m * p.P + col0 + (int64_t)u8 * 8, h);
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) h[k] = __float2half_rn(0.f);
            }
            uint4 v;
            __half2 h01 = __halves2half2(h[0], h[1]), h23 = __halves2half2(h[2], h[3]);
            __half2 h45 = __halves2half2(h[4], h[5]), h67 = __halves2half2(h[6], h[7]);
            v.x = *reinterpret_cast<uint32_t *>(&h01); v.y = *reinterpret_cast<uint32_t *>(&h23);
            v.z = *reinterpret_cast<uint32_t *>(&h45); v.w = *reinterpret_cast<uint32_t *>(&h67);
            *reinterpret_cast<uint4 *>(xs + xs_index(u8 * 8, m, MP)) = v;
        }
        __syncthreads();
        for (int m = warp; m < p.M; m += NWARP) {                       // fixed-order sums: same bits every run
            float s = 0.f;
            for (int c = lane; c < NC * KC; c += 32) s += __half2float(xs[xs_index(c, m, MP)]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) tt.sumx[m] = s;
        }
        __syncthreads();
    }

    // ---- 4. stream the tiles
    float *out = p.S > 1 ? p.part + (int64_t)split * p.M * p.Q : p.Y;
    const uint32_t xs_u32 = smem_u32(xs);
    const int g = lane >> 2, t = lane & 3;
    float acc[NT][4];
    for (int u = 0; u < units; ++u) {
        if (u + NST - 1 < units) issue(u + NST - 1);
        cp_async_commit();
        cp_async_wait<NST - 1>();
        __syncwarp();
        const int tile = warp + (u / NC) * NWARP, chunk = u - (u / NC) * NC;
        const int nb = tt.tile_nb[tile];
        if (chunk == 0) {
#pragma unroll
            for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
        }
        const uint32_t stage = ring_w + (u % NST) * STAGE_BYTES;
        const uint32_t xs_chunk = xs_u32 + (uint32_t)(chunk * 16 * p.MP * 16);
        switch (nb) {                                                   // warp-uniform
            case 8: chunk_mma<8, NT>(stage, xs_chunk, p.MP, lane, acc); break;
            case 7: chunk_mma<7, NT>(stage, xs_chunk, p.MP, lane, acc); break;
            case 6: chunk_mma<6, NT>(stage, xs_chunk, p.MP, lane, acc); break;
            case 5: chunk_mma<5, NT>(stage, xs_chunk, p.MP, lane, acc); break;
            case 4: chunk_mma<4, NT>(stage, xs_chunk, p.MP, lane, acc); break;
            case 3: chunk_mma<3, NT>(stage, xs_chunk, p.MP, lane, acc); break;
            default: break;
        }
        if (chunk == NC - 1) {
            if (nb != 0) {
                // y = tau_s * sum(x * id) + min_s * sum(x); thread holds rows g, g+8 and tokens 8n+2t, 8n+2t+1
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int rr = g + 8 * hrow;
                    const int q = tt.row[tile][rr];
                    if (q >= 0) {
                        const float ms = tt.ms[tile][rr], ts = tt.ts[tile][rr];
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const int m = 8 * n + 2 * t + k;
                                if (m < p.M) out[(int64_t)m * p.Q + q] = __fmaf_rn(ts, acc[n][2 * hrow + k], ms * tt.sumx[m]);
                            }
                        }
                    }
                }
            } else {
                // per-element class: rows the fragment path cannot read (width outside 3..8, or a row that does not
                // start on a 16-byte boundary).  One row at a time, ids byte-wise from global memory.
                for (int rr = 0; rr < tt.tile_cnt[tile]; ++rr) {
                    const int q = tt.row[tile][rr];
                    const int rnb = __ldg(p.nbits + q);
                    const int64_t base = __ldg(p.bit_off + q) + (int64_t)kc0 * KC * rnb;
                    const float ms = tt.ms[tile][rr], ts = tt.ts[tile][rr];
                    for (int m0 = 0; m0 < p.M; m0 += 8) {
                        float a[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) a[k] = 0.f;
                        for (int c = lane; c < NC * KC; c += 32) {
                            const float wv = band(field_bytes(p.ids, base + (int64_t)c * rnb, rnb), ts, ms);
#pragma unroll
                            for (int k = 0; k < 8; ++k)
                                if (m0 + k < p.M) a[k] = __fmaf_rn(__half2float(xs[xs_index(c, m0 + k, p.MP)]), wv, a[k]);
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) a[k] += __shfl_xor_sync(0xffffffffu, a[k], o);
                            if (lane == 0 && m0 + k < p.M) out[(int64_t)(m0 + k) * p.Q + q] = a[k];
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();

    // ---- 5. K-ranges: the last CTA of the row block adds the partial sums in range order
    if (p.S > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int old = atomicAdd(p.ticket + blockIdx.x, 1);
            tt.is_last = old == p.S - 1;
        }
        __syncthreads();
        if (tt.is_last) {
            __threadfence();
            for (int idx = tid; idx < p.M * nrows; idx += NWARP * 32) {
                const int m = idx / nrows, r = idx - m * nrows;
                const int64_t o = (int64_t)m * p.Q + q0 + r;
                float s = 0.f;
                for (int k = 0; k < p.S; ++k) s += __ldcg(p.part + (int64_t)k * p.M * p.Q + o);
                p.Y[o] = s;
            }
            if (tid == 0) p.ticket[blockIdx.x] = 0;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// host side

struct Plan {
    int nblk, S, nc_per, nc_total, MP, NT;
    size_t xs_bytes, smem_bytes;
    int64_t part_bytes, ticket_bytes;
};

static int device_sms() {
    static thread_local int dev_cached = -1, n = 148;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != dev_cached) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { cudaGetLastError(); n = 148; }
        dev_cached = dev;
    }
    return n;
}

static Plan make_plan(int64_t M, int64_t Q, int64_t P) {
    Plan pl{};
    pl.nblk = (int)((Q + RB - 1) / RB);
    pl.nc_total = (int)(P / KC);
    pl.NT = (int)((M + 7) / 8);
    pl.MP = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8 * pl.NT;
    // K-range length: bounded by the shared memory the staged activations may take ...
    int nc_max = XS_MAX_BYTES / (KC * pl.MP * 2);
    if (nc_max < 1) nc_max = 1;
    int S = (pl.nc_total + nc_max - 1) / nc_max;
    // ... and short enough that the grid fills the GPU about three times over, but not below 4 chunks per range
    const int want = (3 * device_sms() + pl.nblk - 1) / (pl.nblk > 0 ? pl.nblk : 1);
    int s_fill = want;
    const int s_cap = pl.nc_total / 4 > 0 ? pl.nc_total / 4 : 1;
    if (s_fill > s_cap) s_fill = s_cap;
    if (S < s_fill) S = s_fill;
    if (S < 1) S = 1;
    if (pl.nblk > MAX_TICKET_BLOCKS) S = (pl.nc_total + nc_max - 1) / nc_max;   // more row blocks than counters
    pl.nc_per = (pl.nc_total + S - 1) / S;
    pl.S = (pl.nc_total + pl.nc_per - 1) / pl.nc_per;                   // no empty range
    pl.xs_bytes = (size_t)pl.nc_per * KC * pl.MP * 2;
    pl.smem_bytes = (size_t)NWARP * NST * STAGE_BYTES + pl.xs_bytes;
    pl.part_bytes = pl.S > 1 ? (int64_t)pl.S * M * Q * 4 : 0;
    pl.part_bytes = (pl.part_bytes + 255) / 256 * 256;
    pl.ticket_bytes = pl.S > 1 ? TICKET_BYTES : 0;
    return pl;
}

static bool fast_layout_ok(const qvb8_pack *w, const void *X, int x_dtype) {
    return w->P > 0 && w->P % KC == 0 && aligned(w->ids, 16) && aligned(X, 16) &&
           (x_dtype != QVB8_F32 || aligned(X, 16));
}

template <int XT, int NT>
static int launch_one(const SmallMParams &prm, const Plan &pl, cudaStream_t st) {
    auto kern = small_m_kernel<XT, NT>;
    static thread_local size_t granted = 0;
    static thread_local int granted_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (pl.smem_bytes > granted || dev != granted_dev) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024)) != cudaSuccess)
            return cuda_status("qvb8_small_m: shared memory opt-in");
        granted = 200 * 1024;
        granted_dev = dev;
    }
    kern<<<dim3(pl.nblk, pl.S), NWARP * 32, pl.smem_bytes, st>>>(prm);
    return cuda_status("qvb8_small_m launch");
}

template <int XT>
static int launch_nt(const SmallMParams &prm, const Plan &pl, cudaStream_t st) {
    switch (pl.NT) {
        case 1: return launch_one<XT, 1>(prm, pl, st);
        case 2: return launch_one<XT, 2>(prm, pl, st);
        case 3: return launch_one<XT, 3>(prm, pl, st);
        case 4: return launch_one<XT, 4>(prm, pl, st);
        case 5: return launch_one<XT, 5>(prm, pl, st);
        default: return launch_one<XT, 6>(prm, pl, st);
    }
}

}  // namespace qv

QV_API int64_t qvb8_small_m_scratch_bytes(int64_t M, int64_t Q, int64_t P) {
    using namespace qv;
    if (M < 1 || M > 48 || Q <= 0 || P <= 0 || P % KC != 0) return 0;
    const Plan pl = make_plan(M, Q, P);
    return pl.part_bytes + pl.ticket_bytes;
}

QV_API int qvb8_small_m(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, float *Y, void *scratch,
                        int64_t scratch_bytes, void *stream) {
    using namespace qv;
    if (int rc = check_small_m_args(w, X, x_dtype, x_mode, M, Y, "qvb8_small_m")) return rc;
    if (w->Q == 0) return QVB8_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (x_mode != 0 || !fast_layout_ok(w, X, x_dtype))
        return launch_small_m_generic(w, X, x_dtype, x_mode, (int)M, Y, st);
    const Plan pl = make_plan(M, w->Q, w->P);
    if (pl.part_bytes + pl.ticket_bytes > 0) {
        if (!scratch || scratch_bytes < pl.part_bytes + pl.ticket_bytes)
            return fail(QVB8_ERR_SCRATCH, "qvb8_small_m: scratch of %lld bytes needed, %lld given",
                        (long long)(pl.part_bytes + pl.ticket_bytes), (long long)scratch_bytes);
        if (!aligned(scratch, 16)) return fail(QVB8_ERR_ALIGN, "qvb8_small_m: scratch must be 16-byte aligned");
    }
    SmallMParams prm{};
    prm.ids = w->ids; prm.min_s = w->min_s; prm.tau_s = w->tau_s; prm.nbits = w->nbits; prm.bit_off = w->bit_off;
    prm.X = X; prm.Y = Y;
    if (pl.S > 1 && pl.nblk > MAX_TICKET_BLOCKS)
        return fail(QVB8_ERR_ARG, "qvb8_small_m: %d row blocks with a split K-range exceed the %d ticket counters",
                    pl.nblk, MAX_TICKET_BLOCKS);
    prm.ticket = reinterpret_cast<int *>(scratch);
    prm.part = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scratch) + TICKET_BYTES);
    prm.Q = (int)w->Q; prm.P = (int)w->P; prm.M = (int)M; prm.MP = pl.MP; prm.S = pl.S; prm.nc_per = pl.nc_per;
    prm.nc_total = pl.nc_total;
    int rc;
    if (x_dtype == QVB8_F16) rc = launch_nt<QVB8_F16>(prm, pl, st);
    else if (x_dtype == QVB8_BF16) rc = launch_nt<QVB8_BF16>(prm, pl, st);
    else rc = launch_nt<QVB8_F32>(prm, pl, st);
    if (rc) return rc;
    return launch_fix_escapes(w, X, x_dtype, x_mode, (int)M, Y, st);
}
