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
// Launches:
//   narrow   X -> saturated fp16, stored tile by tile in the order the tensor cores read it (256 tokens x 64 columns =
//            32 KB contiguous: [8-column group][token][8 values]), plus partial sums of the narrowed values
//   main     a CTA owns 128 * NACC output rows (in the plan's width-sorted order) and 256 tokens; K advances in blocks
//            of 64 columns through a ring of shared-memory stages.  Warp roles:
//              warps 0..7  unpack: a thread owns one row; per K block it reads the row's 64 ids (8 * nb bytes, 8-byte
//                          aligned), turns pairs into fp16 integers with shift / mask / or 0x6400 / subtract 1024 and
//                          stores eight 16-byte rows of core matrices (K-major, no swizzle); the next block's words are
//                          already in registers
//              warp 8      one thread: one 32 KB bulk copy per stage for the activations
//              warp 9      one thread: waits for both halves of a stage, issues 4 * NACC tcgen05.mma (128 x 256 x 16)
//                          and commits them to the stage's "empty" barrier
//            At the end the eight unpack warps read the accumulators with tcgen05.ld, apply tau_s, min_s * sum(x) and
//            write Y.
//   wide, escapes   the corrections described above
//
// Waits are bounded: a wait that runs out raises an abort flag and the error word, everybody falls through, copies in
// flight are given time to land, and the tensor memory is released before the CTA exits.
#include "common.cuh"
#include "plan.cuh"

namespace qv {

constexpr int PF_TOK = 256;                // tokens per CTA = MMA N
constexpr int PF_BK = 64;                  // columns per stage
constexpr int PF_UNPACK = 256;             // unpack threads (warps 0..7)
constexpr int PF_THREADS = PF_UNPACK + 64; // + copy warp + MMA warp
constexpr int PF_A_HALF = 128 * PF_BK * 2; // 16 KB: 128 rows of one accumulator
constexpr int PF_B_BYTES = PF_TOK * PF_BK * 2;      // 32 KB
constexpr int PF_SPIN = 1 << 22;
constexpr int PF_KS = 8;                   // column ranges of the partial activation sums
constexpr int PF_EXACT_BITS = 11;          // ids up to this width are exact in fp16
constexpr int PF_MAX_STAGES = 4;
constexpr int PF_WORDS = 10;               // 64-bit words of 64 ids of the widest row unpacked word-wise

__device__ int g_prefill_error = 0;

__device__ __forceinline__ uint32_t pf_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool pf_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    return ok != 0;
}
__device__ __noinline__ bool pf_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
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
__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    if (pf_try_wait(bar, parity)) return true;
    return pf_wait_slow(bar, parity, abort_flag, code);
}
__device__ __forceinline__ void pf_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes stored as 128 contiguous
// bytes; `sbo` bytes between core matrices along the rows, `lbo` bytes between core matrices along K; version 1.
__device__ __forceinline__ uint64_t pf_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

// Position (in halves) of activation (token n, column c) in the tiled fp16 copy; nkb = P / 64.
__host__ __device__ __forceinline__ int64_t x16_index(int n, int c, int nkb) {
    return ((((int64_t)(n >> 8) * nkb + (c >> 6)) * 8 + ((c >> 3) & 7)) * PF_TOK + (n & 255)) * 8 + (c & 7);
}

struct PrefillParams {
    const uint8_t *ids;
    const float *min_s, *tau_s;
    const uint8_t *nbits;
    const int64_t *bit_off;
    const TileDesc *tiles;     // the plan's width-sorted row order, 16 rows per entry
    int max_tiles;
    const __half *X16;         // tiled saturated fp16 copy of X, tokens padded to a multiple of 256 with zeros
    const float *sumx;         // (PF_KS, Mpad) partial sums of the narrowed activations
    float *Y;                  // (M, Q)
    int Q, P, M, Mpad;
};

// The output row of a slot of the plan's order, -1 for padding.
__device__ __forceinline__ int slot_row(const PrefillParams &p, int slot) {
    if ((slot >> 4) >= p.max_tiles) return -1;
    const TileDesc *td = p.tiles + (slot >> 4);
    return (slot & 15) < __ldg(&td->cnt) ? __ldg(&td->row[slot & 15]) : -1;
}

// 64 ids of one row (NB 64-bit words) -> eight 16-byte groups of fp16 integers, group j at dst + j * 2048.
template <int NB>
__device__ __forceinline__ void unpack_row64(const uint64_t (&w)[PF_WORDS], uint8_t *dst) {
    constexpr uint32_t m = (1u << NB) - 1u;
    const __half2 k1024 = __halves2half2(__ushort_as_half((unsigned short)0x6400), __ushort_as_half((unsigned short)0x6400));
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        uint32_t h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = g * 8 * NB + 2 * i * NB;       // first bit of the pair within the row's 64 * NB bits
            const int idx = s >> 5, sh = s & 31;
            const uint32_t lo32 = (idx & 1) ? (uint32_t)(w[idx >> 1] >> 32) : (uint32_t)w[idx >> 1];
            uint32_t t;
            if (sh == 0) t = lo32;
            else if (sh + 2 * NB <= 32) t = lo32 >> sh;
            else {
                const int i2 = idx + 1;
                const uint32_t hi32 = (i2 & 1) ? (uint32_t)(w[i2 >> 1] >> 32) : (uint32_t)w[i2 >> 1];
                t = __funnelshift_r(lo32, hi32, sh);
            }
            const uint32_t u = (t & m) | (((t >> NB) & m) << 16) | 0x64006400u;      // two fp16 numbers 1024 + id
            const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&u), k1024);
            h[i] = *reinterpret_cast<const uint32_t *>(&v);
        }
        *reinterpret_cast<uint4 *>(dst + g * 2048) = make_uint4(h[0], h[1], h[2], h[3]);
    }
}

template <int NACC>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(const PrefillParams p) {
    constexpr int ROWS = 128 * NACC;
    constexpr int A_BYTES = PF_A_HALF * NACC;
    constexpr int STAGE = A_BYTES + PF_B_BYTES;
    constexpr int NSTG = NACC == 2 ? 3 : 4;
    constexpr int GROUPS = 2 / NACC;                    // unpack groups of ROWS threads; group g takes K blocks kb % GROUPS == g
    constexpr uint32_t TMEM_COLS = 256 * NACC;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ alignas(8) uint64_t a_full[PF_MAX_STAGES];     // the unpack warps have written the stage's weights
    __shared__ alignas(8) uint64_t b_full[PF_MAX_STAGES];     // the stage's activations have landed
    __shared__ alignas(8) uint64_t empty[PF_MAX_STAGES];      // the MMAs that read the stage have completed
    __shared__ alignas(8) uint64_t all_done;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_word;
    __shared__ float sx[PF_TOK];                              // sum of the narrowed activations of each token of the tile
    volatile int *abort_flag = &abort_word;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot0 = blockIdx.x * ROWS;                // first row slot (plan order) of this CTA
    const int n0 = blockIdx.y * PF_TOK;
    // surplus tiles at the end of the plan's table are empty: a CTA that starts in them has no rows at all
    if ((slot0 >> 4) >= p.max_tiles || __ldg(&p.tiles[slot0 >> 4].cnt) == 0) return;
    if (tid == 0) {
        for (int s = 0; s < NSTG; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(pf_smem(&a_full[s])), "r"(4 * NACC) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&b_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&empty[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&all_done)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_word = 0;
    }
    if (warp == 0) {                                    // one warp allocates (and later frees) the tensor-memory columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(pf_smem(&tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid < PF_TOK) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < PF_KS; ++k) t += __ldg(p.sumx + (int64_t)k * p.Mpad + n0 + tid);
        sx[tid] = t;
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base;
    const int nkb = p.P / PF_BK;

    if (warp < 8) {
        // ------------------------------------------------------------------------------------------ unpack warps
        const int grp = tid / ROWS;                     // 0 for NACC = 2
        const int r = tid % ROWS;                       // row of the CTA's tile
        const int row = slot_row(p, slot0 + r);
        const int nb = row >= 0 ? __ldg(p.nbits + row) : 0;
        const int64_t bit0 = row >= 0 ? __ldg(p.bit_off + row) : 0;
        // mode 0: nothing to contract (padding, or a row wider than fp16 holds exactly: recomputed afterwards)
        // mode 1: whole 64-bit words, widths 1..10;  mode 2: id by id
        const bool words_ok = (bit0 & 63) == 0 && (reinterpret_cast<uintptr_t>(p.ids) & 7) == 0 && nb >= 1 && nb <= 10;
        const int mode = (row < 0 || nb > PF_EXACT_BITS || nb < 1) ? 0 : (words_ok ? 1 : 2);
        const uint64_t *wrow = reinterpret_cast<const uint64_t *>(p.ids + (bit0 >> 3));
        uint8_t *const dst_row = smem + (r >> 7) * PF_A_HALF + (r & 127) * 16;

        uint64_t w[PF_WORDS];
#pragma unroll
        for (int i = 0; i < PF_WORDS; ++i) w[i] = 0;
        if (mode == 1 && grp < nkb) {
#pragma unroll
            for (int i = 0; i < PF_WORDS; ++i)
                if (i < nb) w[i] = __ldg(wrow + (int64_t)grp * nb + i);
        }
        bool alive = true;
        for (int kb = grp; kb < nkb && alive; kb += GROUPS) {
            const int s = kb % NSTG, u = kb / NSTG;
            uint64_t nx[PF_WORDS];
#pragma unroll
            for (int i = 0; i < PF_WORDS; ++i) nx[i] = 0;
            if (mode == 1 && kb + GROUPS < nkb) {        // the next block's words travel while this one is unpacked
#pragma unroll
                for (int i = 0; i < PF_WORDS; ++i)
                    if (i < nb) nx[i] = __ldg(wrow + (int64_t)(kb + GROUPS) * nb + i);
            }
            if (u > 0) alive = pf_wait(pf_smem(&empty[s]), (u - 1) & 1, abort_flag, 21);
            if (!alive) break;
            uint8_t *dst = dst_row + s * STAGE;
            if (mode == 1) {
                switch (nb) {
                case 1: unpack_row64<1>(w, dst); break;
                case 2: unpack_row64<2>(w, dst); break;
                case 3: unpack_row64<3>(w, dst); break;
                case 4: unpack_row64<4>(w, dst); break;
                case 5: unpack_row64<5>(w, dst); break;
                case 6: unpack_row64<6>(w, dst); break;
                case 7: unpack_row64<7>(w, dst); break;
                case 8: unpack_row64<8>(w, dst); break;
                case 9: unpack_row64<9>(w, dst); break;
                default: unpack_row64<10>(w, dst); break;
                }
            } else if (mode == 2) {
                for (int g = 0; g < 8; ++g) {
                    uint32_t h[4];
                    for (int i = 0; i < 4; ++i) {
                        const int col = kb * PF_BK + g * 8 + 2 * i;
                        const uint32_t a0 = field_bytes(p.ids, bit0 + (int64_t)col * nb, nb);
                        const uint32_t a1 = field_bytes(p.ids, bit0 + (int64_t)(col + 1) * nb, nb);
                        const __half2 hh = __halves2half2(__ushort2half_rn((unsigned short)a0), __ushort2half_rn((unsigned short)a1));
                        h[i] = *reinterpret_cast<const uint32_t *>(&hh);
                    }
                    *reinterpret_cast<uint4 *>(dst + g * 2048) = make_uint4(h[0], h[1], h[2], h[3]);
                }
            } else {
#pragma unroll
                for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4 *>(dst + g * 2048) = make_uint4(0u, 0u, 0u, 0u);
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // generic-proxy writes -> visible to the MMA
            __syncwarp();
            if (lane == 0) pf_arrive(pf_smem(&a_full[s]));
#pragma unroll
            for (int i = 0; i < PF_WORDS; ++i) w[i] = nx[i];
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------------------------------------ activation copies
        if (lane == 0) {
            const uint8_t *src = reinterpret_cast<const uint8_t *>(p.X16) + (int64_t)blockIdx.y * nkb * PF_B_BYTES;
            bool alive = true;
            for (int kb = 0; kb < nkb && alive; ++kb) {
                const int s = kb % NSTG, u = kb / NSTG;
                if (u > 0) alive = pf_wait(pf_smem(&empty[s]), (u - 1) & 1, abort_flag, 22);
                if (!alive) break;
                const uint32_t bar = pf_smem(&b_full[s]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"((uint32_t)PF_B_BYTES) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                             :: "r"(pf_smem(smem + s * STAGE + A_BYTES)), "l"(src + (int64_t)kb * PF_B_BYTES), "r"((uint32_t)PF_B_BYTES), "r"(bar)
                             : "memory");
            }
        }
    } else {
        // ------------------------------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, fp16 x fp16, both operands K-major, N = 256, M = 128
            constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(PF_TOK >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            bool alive = true;
            for (int kb = 0; kb < nkb && alive; ++kb) {
                const int s = kb % NSTG, u = kb / NSTG;
                alive = pf_wait(pf_smem(&a_full[s]), u & 1, abort_flag, 23);
                if (alive) alive = pf_wait(pf_smem(&b_full[s]), u & 1, abort_flag, 24);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t a32 = pf_smem(smem + s * STAGE), b32 = a32 + A_BYTES;
#pragma unroll
                for (int h = 0; h < NACC; ++h) {
#pragma unroll
                    for (int kk = 0; kk < PF_BK / 16; ++kk) {
                        // one MMA covers two 8-column groups: core matrices 2 kk and 2 kk + 1 along K
                        const uint64_t da = pf_desc(a32 + h * PF_A_HALF + 2 * kk * 2048, 2048, 128);
                        const uint64_t db = pf_desc(b32 + 2 * kk * (PF_TOK * 16), PF_TOK * 16, 128);
                        const uint32_t accumulate = (kb > 0 || kk > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                            " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n"
                            :: "r"(tmem + (uint32_t)(h * 256)), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
                            : "memory");
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(pf_smem(&empty[s])) : "memory");
                if (kb == nkb - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(pf_smem(&all_done)) : "memory");
            }
        }
    }

    // ---- epilogue: tensor memory -> registers -> Y.  A warp reads the 32 lanes (warp & 3) * 32 ...; with two
    // accumulators warps 4..7 take the second, with one they take the upper 128 tokens.
    if (warp < 8) {
        bool alive = !*abort_flag;
        if (alive) alive = pf_wait(pf_smem(&all_done), 0, abort_flag, 25);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (alive) {
            const int lq = (warp & 3) * 32;
            const int h = NACC == 2 ? (warp >> 2) : 0;
            const int cbeg = NACC == 2 ? 0 : (warp >> 2) * 128, cend = NACC == 2 ? 256 : cbeg + 128;
            const int row = slot_row(p, slot0 + h * 128 + lq + lane);
            const float ts = row >= 0 ? __ldg(p.tau_s + row) : 0.f, ms = row >= 0 ? __ldg(p.min_s + row) : 0.f;
            for (int c0 = cbeg; c0 < cend; c0 += 32) {
                uint32_t d[32];
                const uint32_t taddr = tmem + ((uint32_t)lq << 16) + (uint32_t)(h * 256 + c0);
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
                    if (row >= 0 && nn < p.M) p.Y[(int64_t)nn * p.Q + row] = __fmaf_rn(ts, __uint_as_float(d[j]), ms * sx[c0 + j]);
                }
            }
        }
    }
    if (*abort_flag && warp == 8) {                      // copies may still be in flight: let them land before the CTA goes
        uint64_t t0, t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        for (int i = 0; i < (1 << 16); ++i) {
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            if (t - t0 > 200000ull) break;
            __nanosleep(1000);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// X (M, P) of any input type -> saturated fp16 in the tiled order, tokens padded to Mpad with zeros, and the sums of
// the narrowed values per token and column range (fixed order: a thread sums its groups in order, then eight warps are
// added in order).  Block = 32 tokens (lane) x 8 warps; blockIdx.y = column range.
__global__ void __launch_bounds__(256) prefill_narrow_kernel(const void *__restrict__ X, int x_dtype, int M, int Mpad, int P,
                                                             __half *__restrict__ X16, float *__restrict__ sumx) {
    __shared__ float part[8][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 32 + lane;
    const int nkb = P / PF_BK, ngrp = P / 8;
    const int per = (ngrp + PF_KS - 1) / PF_KS;
    const int g0 = blockIdx.y * per, g1 = min(ngrp, g0 + per);
    float s = 0.f;
    for (int g = g0 + warp; g < g1; g += 8) {
        __half h[8];
        if (n < M) {
            const int64_t i = (int64_t)n * P + g * 8;
            if (x_dtype == QVB8_F32) {
                const float4 a = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(X) + i));
                const float4 b = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(X) + i) + 1);
                h[0] = sat_half(a.x); h[1] = sat_half(a.y); h[2] = sat_half(a.z); h[3] = sat_half(a.w);
                h[4] = sat_half(b.x); h[5] = sat_half(b.y); h[6] = sat_half(b.z); h[7] = sat_half(b.w);
            } else if (x_dtype == QVB8_BF16) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(X) + i));
                const __nv_bfloat16 *b = reinterpret_cast<const __nv_bfloat16 *>(&v);
#pragma unroll
                for (int k = 0; k < 8; ++k) h[k] = sat_half(__bfloat162float(b[k]));
            } else {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(X) + i));
                const __half *b = reinterpret_cast<const __half *>(&v);
#pragma unroll
                for (int k = 0; k < 8; ++k) h[k] = sat_half(__half2float(b[k]));
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) s += __half2float(h[k]);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) h[k] = __float2half_rn(0.f);
        }
        *reinterpret_cast<uint4 *>(X16 + x16_index(n, g * 8, nkb)) = *reinterpret_cast<const uint4 *>(h);
    }
    part[warp][lane] = s;
    __syncthreads();
    if (warp == 0) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += part[k][lane];
        sumx[(int64_t)blockIdx.y * Mpad + n] = t;
    }
}

// Y[m, q] += sum over the escapes of row q of x16[m, col] * (exact - band), in stored order
__global__ void __launch_bounds__(256) prefill_escapes_kernel(const int *__restrict__ esc_ptr, const int *__restrict__ esc_col,
                                                              const float *__restrict__ esc_delta, const __half *__restrict__ X16,
                                                              float *__restrict__ Y, int Q, int P, int M) {
    const int q = blockIdx.x;
    const int e0 = __ldg(esc_ptr + q), e1 = __ldg(esc_ptr + q + 1);
    if (e0 == e1) return;
    const int nkb = P / PF_BK;
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        float a = 0.f;
        for (int e = e0; e < e1; ++e) a = __fmaf_rn(__half2float(X16[x16_index(m, __ldg(esc_col + e), nkb)]), __ldg(esc_delta + e), a);
        Y[(int64_t)m * Q + q] += a;
    }
}

// Rows wider than 11 bits: their ids are not exact in fp16 (integers above 2048 are not all representable), so the
// tensor-core result of such a row is replaced by an fp32 product over the row.  They are rare (rows dominated by
// outliers).  First a compact list of them, then one warp per (wide row, token).
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
    const int nkb = p.P / PF_BK;
    for (int wi = blockIdx.x; wi < n; wi += gridDim.x) {
        const int q = list[wi];
        const int nb = __ldg(p.nbits + q);
        const int64_t bit0 = __ldg(p.bit_off + q);
        const float ts = __ldg(p.tau_s + q), ms = __ldg(p.min_s + q);
        float a = 0.f;
        for (int c = lane; c < p.P; c += 32)
            a = __fmaf_rn(__half2float(p.X16[x16_index(m, c, nkb)]), band(field_bytes(p.ids, bit0 + (int64_t)c * nb, nb), ts, ms), a);
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

static int g_prefill_rows = 0;      // tuning: 0 = choose, 128 / 256 = rows per CTA

template <int NACC>
static int launch_prefill(const PrefillParams &prm, cudaStream_t st) {
    constexpr int STAGE = PF_A_HALF * NACC + PF_B_BYTES;
    constexpr int NSTG = NACC == 2 ? 3 : 4;
    constexpr int SMEM = NSTG * STAGE + 1024;
    static thread_local int granted_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != granted_dev) {
        if (cudaFuncSetAttribute(prefill_kernel<NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return cuda_status("qvb8_prefill: shared memory opt-in");
        granted_dev = dev;
    }
    const int slots = prm.max_tiles * 16;
    const dim3 grid((unsigned)((slots + 128 * NACC - 1) / (128 * NACC)), (unsigned)(prm.Mpad / PF_TOK));
    prefill_kernel<NACC><<<grid, PF_THREADS, SMEM, st>>>(prm);
    return cuda_status("qvb8_prefill");
}

}  // namespace qv

QV_API void qvb8_prefill_set_tuning(int rows_per_cta) { qv::g_prefill_rows = rows_per_cta; }

QV_API int64_t qvb8_prefill_scratch_bytes(int64_t M, int64_t Q, int64_t P) {
    if (M <= 0 || P <= 0 || Q < 0) return 0;
    const int64_t Mpad = (M + qv::PF_TOK - 1) / qv::PF_TOK * qv::PF_TOK;
    return qv::up256(Mpad * P * 2) + qv::up256(qv::PF_KS * Mpad * 4) + qv::up256((Q + 1) * 4);
}

QV_API int qvb8_prefill(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int64_t M, float *Y, void *scratch,
                        int64_t scratch_bytes, void *stream) {
    using namespace qv;
    if (int rc = check_pack(w, "qvb8_prefill")) return rc;
    if (int rc = check_device("qvb8_prefill")) return rc;
    if (!X || !Y || M <= 0 || M > 0x7fffff00) return fail(QVB8_ERR_ARG, "qvb8_prefill: bad X / Y / M");
    if (x_dtype != QVB8_F16 && x_dtype != QVB8_BF16 && x_dtype != QVB8_F32) return fail(QVB8_ERR_ARG, "qvb8_prefill: bad X dtype");
    if (w->Q == 0) return QVB8_OK;
    if (w->P % PF_BK != 0) return fail(QVB8_ERR_ARG, "qvb8_prefill: P must be a multiple of %d", PF_BK);
    if (!aligned(X, 16)) return fail(QVB8_ERR_ARG, "qvb8_prefill: X must be 16-byte aligned");
    if (!plan || !aligned(plan, 256)) return fail(QVB8_ERR_ARG, "qvb8_prefill: the pack's plan is needed (qvb8_plan_build), 256-byte aligned");
    const int64_t need = qvb8_prefill_scratch_bytes(M, w->Q, w->P);
    if (!scratch || scratch_bytes < need || !aligned(scratch, 256))
        return fail(QVB8_ERR_SCRATCH, "qvb8_prefill: scratch of %lld bytes (256-byte aligned) needed, %lld given", (long long)need, (long long)scratch_bytes);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int64_t Mpad = (M + PF_TOK - 1) / PF_TOK * PF_TOK;
    uint8_t *sc = reinterpret_cast<uint8_t *>(scratch);
    __half *X16 = reinterpret_cast<__half *>(sc);
    float *sumx = reinterpret_cast<float *>(sc + up256(Mpad * w->P * 2));
    int *wide = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(sumx) + up256(PF_KS * Mpad * 4));      // [0] count, then rows
    prefill_narrow_kernel<<<dim3((unsigned)(Mpad / 32), PF_KS), 256, 0, st>>>(X, x_dtype, (int)M, (int)Mpad, (int)w->P, X16, sumx);
    if (int rc = cuda_status("qvb8_prefill narrow")) return rc;

    const PlanLayout L = plan_layout(w->Q, w->n_esc);
    const uint8_t *pb = reinterpret_cast<const uint8_t *>(plan);
    PrefillParams prm{w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, reinterpret_cast<const TileDesc *>(pb + L.tiles), L.max_tiles,
                      X16, sumx, Y, (int)w->Q, (int)w->P, (int)M, (int)Mpad};
    // rows per CTA: 256 halves the activation traffic per SM; 128 gives twice as many CTAs.  Take the one whose last
    // wave wastes less (a 256-row CTA takes twice as long; a 128-row one is charged 15 % for the extra traffic).
    int sms = 148;
    {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int64_t tok_tiles = Mpad / PF_TOK;
    const int64_t c256 = ((int64_t)L.max_tiles * 16 + 255) / 256 * tok_tiles, c128 = ((int64_t)L.max_tiles * 16 + 127) / 128 * tok_tiles;
    const double t256 = (double)((c256 + sms - 1) / sms) * 2.0, t128 = (double)((c128 + sms - 1) / sms) * 1.15;
    const int rows = g_prefill_rows ? g_prefill_rows : (t256 <= t128 ? 256 : 128);
    if (int rc = rows == 256 ? launch_prefill<2>(prm, st) : launch_prefill<1>(prm, st)) return rc;

    if (cudaMemsetAsync(wide, 0, sizeof(int), st) != cudaSuccess) return cuda_status("qvb8_prefill memset");
    prefill_wide_list_kernel<<<(unsigned)((w->Q + 255) / 256), 256, 0, st>>>(w->nbits, (int)w->Q, wide + 1, wide);
    prefill_wide_rows_kernel<<<dim3(64, (unsigned)((M + 7) / 8)), 256, 0, st>>>(prm, wide + 1, wide);
    if (int rc = cuda_status("qvb8_prefill wide rows")) return rc;
    if (w->n_esc > 0) {
        prefill_escapes_kernel<<<(unsigned)w->Q, 256, 0, st>>>(reinterpret_cast<const int *>(pb + L.esc_ptr), reinterpret_cast<const int *>(pb + L.esc_col),
                                                              reinterpret_cast<const float *>(pb + L.esc_delta), X16, Y, (int)w->Q, (int)w->P, (int)M);
        if (int rc = cuda_status("qvb8_prefill escapes")) return rc;
    }
    return QVB8_OK;
}
