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
//   main     a CTA owns 128 output rows (in the plan's width-sorted order) and 256 tokens; K advances in blocks of 64
//            columns.  The weights reach the tensor cores through TENSOR MEMORY (tcgen05.mma with the A operand in
//            tensor memory), so shared memory carries only the activations and the packed ids:
//              unpack warps (PF_G groups of four; three by default).  A thread owns one row = one lane of tensor
//                          memory; group g takes the pairs of K blocks g, g + PF_G, ...  A warp fetches its own 32
//                          rows x 128 ids with 16-byte cp.async (eight lanes per row: whole lines, not one line per
//                          lane) into a private buffer whose row stride is an odd multiple of 16 bytes; then every
//                          thread reads its row (nb 16-byte vectors), turns pairs of ids into fp16 integers (one
//                          window, mask | 0x6400.., one HFMA2 for 6..8 bits) and stores 2 x 32 registers with
//                          tcgen05.st into its lane of one of four 64-column weight slots
//              copy warp   one thread: one 32 KB bulk copy per K block for the activations (four stages, freed in pairs)
//              MMA warp    one thread: waits for a weight slot and an activation stage, issues four tcgen05.mma
//                          (128 x 256 x 16, accumulator in columns 0..255) per K block and, per pair of K blocks,
//                          commits them to the barriers that free the two stages and the slot
//            At the end eight of the unpack warps read the accumulator with tcgen05.ld, apply tau_s, min_s * sum(x)
//            and write Y.
//   wide, escapes   the corrections described above
//
// Waits are bounded: a wait that runs out raises an abort flag and the error word, everybody falls through, copies in
// flight are given time to land, and the tensor memory is released before the CTA exits.
#include "common.cuh"
#include "plan.cuh"

namespace qv {

constexpr int PF_TOK = 256;                // tokens per CTA = MMA N
constexpr int PF_BK = 64;                  // columns per stage
#ifndef QVB8_PF_GROUPS
#define QVB8_PF_GROUPS 3
#endif
constexpr int PF_G = QVB8_PF_GROUPS;       // unpack groups of four warps (a group owns whole pairs of K blocks)
constexpr int PF_UW = 4 * PF_G;            // unpack warps
constexpr int PF_UNPACK = 32 * PF_UW;      // unpack threads
constexpr int PF_THREADS = PF_UNPACK + 64; // + copy warp + MMA warp
constexpr int PF_NBUF = PF_G <= 2 ? 2 : 1; // buffers of packed ids per unpack warp
constexpr int PF_EG = PF_G >= 4 ? 4 : 2;   // groups of four warps that share the epilogue
// registers: the allocation is per four warps, so 14 warps (three groups) may use 128 each, 18 warps only 96
constexpr int PF_B_BYTES = PF_TOK * PF_BK * 2;      // 32 KB
constexpr int PF_SPIN = 1 << 22;
constexpr int PF_KS = 8;                   // column ranges of the partial activation sums
constexpr int PF_EXACT_BITS = 11;          // ids up to this width are exact in fp16
constexpr int PF_NBS = 4;                  // activation stages in shared memory (even: they are freed in pairs)
constexpr int PF_NU = 4;                   // weight units (pairs of K blocks, 64 columns) in tensor memory
constexpr int PF_VECS = 8;                 // 16-byte vectors of a pair of K blocks (128 ids) of the widest row that is copied
constexpr int PF_RAW_BUF = 32 * 16 * (PF_VECS | 1);   // bytes of one warp's buffer for a pair at the widest row stride
constexpr int PF_TMEM_COLS = 512;          // 256 accumulator columns + PF_NU * 64 weight columns
constexpr int PF_SMEM = PF_NBS * PF_B_BYTES + PF_UW * PF_NBUF * PF_RAW_BUF + 1024;

__device__ int g_prefill_error = 0;

__device__ __forceinline__ uint32_t pf_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool pf_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    return ok != 0;
}
__device__ __noinline__ bool pf_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code, unsigned backoff_ns) {
    uint64_t t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (int i = 0; i < PF_SPIN; ++i) {
        if (pf_try_wait(bar, parity)) return true;
        if (backoff_ns) __nanosleep(backoff_ns);         // a polling warp takes issue slots from the unpack warps of its scheduler
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
__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code, unsigned backoff_ns = 0) {
    if (pf_try_wait(bar, parity)) return true;
    return pf_wait_slow(bar, parity, abort_flag, code, backoff_ns);
}
// Polling wait (tuning switch 64) for the single threads whose wake-up latency is on the critical path (MMA issue,
// activation copies): mbarrier.test_wait never suspends the thread.  Bounded like pf_wait.  Measured slower than the
// suspending wait (0.63 against 0.50 ms per call on 5120 x 17408 x 2048): the polling warps take issue slots.
__device__ __noinline__ bool pf_wait_poll(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    uint64_t t0 = 0;
    for (int i = 0; i < (1 << 28); ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 255) == 255) {
            if (*abort_flag) return false;
            uint64_t t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            if (t - t0 > 2000000000ull) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_prefill_error, 0, code);
    return false;
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

// Position (in halves) of activation (token n, column c) in the tiled fp16 copy; nkb = P / 64.  Inside every group of
// four columns the order is 0, 2, 1, 3: the unpack threads build fp16 pairs from ids two columns apart (for 6..8-bit
// rows such a pair comes out of ONE 32-bit window), so a 32-bit operand register holds columns (k, k + 2) and the
// activations follow the same order.
__host__ __device__ __forceinline__ int pair_order(int a) { return (((a >> 1) ^ a) & 1) ? (a ^ 3) : a; }
__host__ __device__ __forceinline__ int64_t x16_index(int n, int c, int nkb) {
    return ((((int64_t)(n >> 8) * nkb + (c >> 6)) * 8 + ((c >> 3) & 7)) * PF_TOK + (n & 255)) * 8 + pair_order(c & 7);
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
    int debug;                 // tuning aid: 1 = no unpack arithmetic, 2 = no activation copies, 4 = no weight fetch, 8 = no tensor-memory stores, 16 = no MMAs, 48 = no MMAs and plain barrier arrivals instead of commits, 64 = polling waits
};

// The output row of a slot of the plan's order, -1 for padding.
__device__ __forceinline__ int slot_row(const PrefillParams &p, int slot) {
    if ((slot >> 4) >= p.max_tiles) return -1;
    const TileDesc *td = p.tiles + (slot >> 4);
    return (slot & 15) < __ldg(&td->cnt) ? __ldg(&td->row[slot & 15]) : -1;
}

// 32-bit word K of the row words held as 16-byte vectors.
template <int K, int NV>
__device__ __forceinline__ uint32_t word32(const uint4 (&q)[NV]) {
    static_assert(K >= 0 && K < 4 * NV, "word outside the pair");
    return (K & 3) == 0 ? q[K >> 2].x : (K & 3) == 1 ? q[K >> 2].y : (K & 3) == 2 ? q[K >> 2].z : q[K >> 2].w;
}

// 32 bits of the pair's bit string such that bit `G` of the string lands at bit `AT` of the result; the caller uses
// the SPAN bits from AT on.
template <int G, int AT, int SPAN, int NV>
__device__ __forceinline__ uint32_t window(const uint4 (&q)[NV]) {
    constexpr int P0 = G - AT;                            // string position of result bit 0
    if constexpr (P0 < 0) return word32<0, NV>(q) << (-P0);
    else {
        constexpr int idx = P0 >> 5, sh = P0 & 31;
        if constexpr (sh == 0) return word32<idx, NV>(q);
        else if constexpr (sh + AT + SPAN <= 32) return word32<idx, NV>(q) >> sh;
        else return __funnelshift_r(word32<idx, NV>(q), word32<idx + 1, NV>(q), sh);
    }
}

// The 64 ids of K block H (0 / 1) of a pair of K blocks -> 32 registers of two fp16 integers each.  Register c holds
// columns k and k + 2, k = 4 * (c >> 1) + (c & 1) (see pair_order).  q holds the 128 ids (NB 16-byte vectors).
//   6..8 bits: ONE window puts id k at bit E = 16 - 2 NB and id k + 2 at bit 16; mask | 0x64006400 gives the fp16
//              numbers 1024 + id * 2^E and 1024 + id; one HFMA2 scales and removes the 1024 (exact)
//   others:    two windows, two masks, one subtraction of 1024
// The shifts and logic operations run on the half-rate integer pipe, which is what bounds this kernel: two instead of
// four of them per pair for the common widths.
// The constants of a width, read once per thread from a shared-memory table through volatile loads: as literals the
// compiler re-creates them with a move in front of every use, which doubles the work of the integer pipe.
struct PairConst {
    uint32_t mask;      // (m << E) | (m << 16) for 6..8 bits; m for the others
    uint32_t mask_hi;   // m << 16
    uint32_t k64;       // 0x64006400
    uint32_t scale;     // half2 (2^-E, 1)
    uint32_t bias;      // half2 (-1024 * 2^-E, -1024)
};
__device__ __forceinline__ PairConst pair_const_of(int nb) {
    const uint32_t m = (1u << nb) - 1u;
    const int e = (nb >= 6 && nb <= 8) ? 16 - 2 * nb : 0;
    PairConst c;
    c.mask = (nb >= 6 && nb <= 8) ? ((m << e) | (m << 16)) : m;
    c.mask_hi = m << 16;
    c.k64 = 0x64006400u;
    const __half2 sc = __floats2half2_rn(1.0f / (float)(1 << e), 1.0f), bi = __floats2half2_rn(-1024.0f / (float)(1 << e), -1024.0f);
    c.scale = *reinterpret_cast<const uint32_t *>(&sc);
    c.bias = *reinterpret_cast<const uint32_t *>(&bi);
    return c;
}

template <int NB, int H, int I = 0>
__device__ __forceinline__ void unpack64(const uint4 (&q)[NB], const PairConst &pc, uint32_t (&out)[32]) {
    if constexpr (I < 32) {
        constexpr int k = 4 * (I >> 1) + (I & 1);
        constexpr int G0 = (H * 64 + k) * NB, G1 = G0 + 2 * NB;
        uint32_t u;
        if constexpr (NB >= 6 && NB <= 8) {
            constexpr int E = 16 - 2 * NB;
            u = (window<G0, E, 16 - E + NB, NB>(q) & pc.mask) | pc.k64;
        } else {
            u = (window<G1, 16, NB, NB>(q) & pc.mask_hi) | ((window<G0, 0, NB, NB>(q) & pc.mask) | pc.k64);
        }
        const __half2 v = __hfma2(*reinterpret_cast<const __half2 *>(&u), *reinterpret_cast<const __half2 *>(&pc.scale),
                                  *reinterpret_cast<const __half2 *>(&pc.bias));
        out[I] = *reinterpret_cast<const uint32_t *>(&v);
        unpack64<NB, H, I + 1>(q, pc, out);
    }
}

// K block H of a row of width NB: the vectors it touches from the warp's buffer, 64 ids to registers.
template <int NB, int H>
__device__ __forceinline__ void unpack_row_half(const uint4 *__restrict__ src, const PairConst &pc, uint32_t (&out)[32]) {
    uint4 q[NB];
    // vectors of half H (a window of the second half may start in the last word of the first)
    constexpr int V0 = H == 0 ? 0 : (NB / 2 > 0 ? NB / 2 - 1 : 0), V1 = H == 0 ? (NB + 1) / 2 + (NB > 1 ? 1 : 0) : NB;
#pragma unroll
    for (int i = V0; i < (V1 < NB ? V1 : NB); ++i) q[i] = src[i];
    unpack64<NB, H>(q, pc, out);
}

// 32 registers -> 32 columns of tensor memory, lane = this thread's lane of the warp's quarter.
__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
           "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
           "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
           "r"(r[30]), "r"(r[31])
        : "memory");
}

// Row of the CTA's tile: output row, width, first byte, and how its ids reach the unpack thread.
//   mode 0: nothing to contract (padding, or a row wider than fp16 holds exactly: recomputed afterwards)
//   mode 1: 16-byte copies into the warp's buffer (widths 1..8, row start 16-byte aligned);  mode 2: id by id from global memory
struct RowInfo { int row, nb, mode; int64_t bit0; };
__device__ __forceinline__ RowInfo row_info(const PrefillParams &p, int slot) {
    RowInfo r;
    r.row = slot_row(p, slot);
    r.nb = r.row >= 0 ? __ldg(p.nbits + r.row) : 0;
    r.bit0 = r.row >= 0 ? __ldg(p.bit_off + r.row) : 0;
    const bool bulk_ok = (r.bit0 & 127) == 0 && (reinterpret_cast<uintptr_t>(p.ids) & 15) == 0 && r.nb >= 1 && r.nb <= PF_VECS;
    r.mode = (r.row < 0 || r.nb > PF_EXACT_BITS || r.nb < 1) ? 0 : (bulk_ok ? 1 : 2);
    return r;
}

// The rare rows that are read id by id (11 bits wide, or not starting on 16 bytes): one K block to registers.
__device__ __noinline__ void unpack_generic(const uint8_t *__restrict__ ids, int64_t bit0, int nb, int kb, uint32_t *out) {
    for (int i = 0; i < 32; ++i) {
        const int col = kb * PF_BK + 4 * (i >> 1) + (i & 1);          // register i holds columns col, col + 2
        const uint32_t a0 = field_bytes(ids, bit0 + (int64_t)col * nb, nb);
        const uint32_t a1 = field_bytes(ids, bit0 + (int64_t)(col + 2) * nb, nb);
        const __half2 hh = __halves2half2(__ushort2half_rn((unsigned short)a0), __ushort2half_rn((unsigned short)a1));
        out[i] = *reinterpret_cast<const uint32_t *>(&hh);
    }
}

// K block H of this thread's pair -> 32 registers.  No tensor-memory access in here: rows of different widths or
// modes diverge inside, and tcgen05.st is a warp-wide instruction that every lane must reach together.
template <int H>
__device__ __forceinline__ void unpack_half(const PrefillParams &p, const RowInfo &me, const uint4 *__restrict__ src, const PairConst &pc,
                                            int kb, int nkb, uint32_t (&out)[32]) {
    if (me.mode == 1) {
        switch (me.nb) {
        case 1: unpack_row_half<1, H>(src, pc, out); break;
        case 2: unpack_row_half<2, H>(src, pc, out); break;
        case 3: unpack_row_half<3, H>(src, pc, out); break;
        case 4: unpack_row_half<4, H>(src, pc, out); break;
        case 5: unpack_row_half<5, H>(src, pc, out); break;
        case 6: unpack_row_half<6, H>(src, pc, out); break;
        case 7: unpack_row_half<7, H>(src, pc, out); break;
        default: unpack_row_half<8, H>(src, pc, out); break;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) out[i] = 0u;
        if (me.mode == 2 && kb < nkb) {                  // through a stack buffer, so that `out` stays in registers
            uint32_t tmp[32];
            unpack_generic(p.ids, me.bit0, me.nb, kb, tmp);
#pragma unroll
            for (int i = 0; i < 32; ++i) out[i] = tmp[i];
        }
    }
}

__global__ void __maxnreg__(PF_G == 2 ? 168 : PF_G == 3 ? 128 : 96) prefill_kernel(const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];         // PF_NBS activation stages, then 8 warps x 2 buffers of packed ids
    __shared__ alignas(8) uint64_t a_full[PF_NU];             // a pair of K blocks of weights is in tensor memory
    __shared__ alignas(8) uint64_t a_empty[PF_NU];            // ... and the MMAs that read it have completed
    __shared__ alignas(8) uint64_t b_full[PF_NBS];            // a stage's activations have landed
    __shared__ alignas(8) uint64_t b_empty[PF_NBS / 2];       // ... and the MMAs that read a PAIR of stages have completed
    __shared__ alignas(8) uint64_t all_done;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_word, nb_max;
    __shared__ const uint8_t *row_src[128];                   // first byte of each row of the tile (mode 1 rows)
    __shared__ int row_nb1[128];                              // its width, 0 unless mode 1
    __shared__ float sx[PF_TOK];                              // sum of the narrowed activations of each token of the tile
    __shared__ PairConst ctab[11];                            // per width, see PairConst
    volatile int *abort_flag = &abort_word;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot0 = blockIdx.x * 128;                 // first row slot (plan order) of this CTA
    const int n0 = blockIdx.y * PF_TOK;
    // surplus tiles at the end of the plan's table are empty: a CTA that starts in them has no rows at all
    if ((slot0 >> 4) >= p.max_tiles || __ldg(&p.tiles[slot0 >> 4].cnt) == 0) return;
    if (tid == 0) {
        for (int s = 0; s < PF_NU; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;\n" ::"r"(pf_smem(&a_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&a_empty[s])) : "memory");
        }
        for (int s = 0; s < PF_NBS; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&b_full[s])) : "memory");
            if (s < PF_NBS / 2) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&b_empty[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(pf_smem(&all_done)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_word = 0;
        nb_max = 0;
        for (int nb = 1; nb <= PF_VECS; ++nb) ctab[nb] = pair_const_of(nb);
    }
    if (warp == 0) {                                    // one warp allocates (and later frees) the tensor-memory columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(pf_smem(&tmem_base)), "r"((uint32_t)PF_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    __syncthreads();
    // the widest copied row fixes the row stride of the warps' buffers
    RowInfo me{};
    if (tid < 128) {
        me = row_info(p, slot0 + tid);
        const int nb1 = me.mode == 1 ? me.nb : 0;
        row_src[tid] = p.ids + (me.bit0 >> 3);
        row_nb1[tid] = nb1;
        const int wmax = __reduce_max_sync(0xffffffffu, nb1);
        if (lane == 0) atomicMax(&nb_max, wmax);
    } else if (tid < PF_UNPACK) {
        me = row_info(p, slot0 + (tid & 127));
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
    const int nunits = (nkb + 1) >> 1;                  // pairs of K blocks
    const int stride = 16 * (nb_max | 1);               // bytes per row in a warp's buffer: an odd multiple of 16

    if (warp < PF_UW) {
        // ------------------------------------------------------------------------------------------ unpack warps
        // group g = warp >> 2 takes the pairs of K blocks u = g, g + PF_G, ...; a thread owns row (warp & 3) * 32 + lane
        const int g = warp >> 2;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 256u;
        uint8_t *const mybuf = smem + PF_NBS * PF_B_BYTES + warp * PF_NBUF * PF_RAW_BUF;
        PairConst pc;
        {
            const volatile PairConst *vc = &ctab[me.mode == 1 ? me.nb : 1];
            pc.mask = vc->mask; pc.mask_hi = vc->mask_hi; pc.k64 = vc->k64; pc.scale = vc->scale; pc.bias = vc->bias;
        }
        // the warp's rows of a pair -> its buffer: eight lanes per row, 16 bytes each; one commit group per pair.  Per-lane constants: this lane's vector of rows 4 pp + lane / 8.
        uint32_t soff[8];
        int step[8];
#pragma unroll
        for (int pp = 0; pp < 8; ++pp) {
            const int rr = (warp & 3) * 32 + pp * 4 + (lane >> 3);
            step[pp] = 16 * row_nb1[rr];
            soff[pp] = (uint32_t)(row_src[rr] - p.ids) + (uint32_t)((lane & 7) * 16);
        }
        const uint32_t dst0 = pf_smem(mybuf) + (uint32_t)((lane >> 3) * stride + (lane & 7) * 16);
        auto fetch = [&](int u_, int b_) {
            if (u_ < nunits && !(p.debug & 4)) {
                const int nkv = min(2, nkb - 2 * u_);
                const uint32_t dst = dst0 + (uint32_t)(b_ * PF_RAW_BUF);
#pragma unroll
                for (int pp = 0; pp < 8; ++pp) {
                    // a last, single K block is 8 * nb bytes: rounded up to 16 (a row is followed by the next row or by
                    // the buffer's 8 bytes of padding)
                    const int nbr = step[pp] >> 4;
                    const int nv = nkv == 2 ? nbr : (8 * nbr + 15) >> 4;
                    const uint8_t *src = p.ids + soff[pp] + (int64_t)u_ * step[pp];
                    if ((lane & 7) < nv)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + (uint32_t)(pp * 4 * stride)), "l"(src) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        };
        fetch(g, 0);
        // every wait result is made warp-uniform: the tensor-memory stores below need the whole warp
        int it = 0;
        for (int u = g; u < nunits; u += PF_G, ++it) {
            const int kb0 = 2 * u;
            const int b = PF_NBUF == 2 ? (it & 1) : 0;
            if (PF_NBUF == 2) {                          // the next pair travels while this one is unpacked
                fetch(u + PF_G, b ^ 1);
                asm volatile("cp.async.wait_group 1;\n" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            }
            __syncwarp();
            const int slot = u & (PF_NU - 1), use = u / PF_NU;
            const uint32_t taddr = lane_base + (uint32_t)(slot * 64);
            const uint4 *src = reinterpret_cast<const uint4 *>(mybuf + b * PF_RAW_BUF + lane * stride);
            uint32_t out[32];
            if (p.debug & 1) {
#pragma unroll
                for (int i = 0; i < 32; ++i) out[i] = 0u;
            } else unpack_half<0>(p, me, src, pc, kb0, nkb, out);
            // only now is the slot needed: the MMAs that read its previous contents must have completed
            bool ok = true;
            if (use > 0) ok = pf_wait(pf_smem(&a_empty[slot]), (use - 1) & 1, abort_flag, 22);
            if (!__all_sync(0xffffffffu, ok)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (!(p.debug & 8)) tmem_store32(taddr, out);
            if (!(p.debug & 1)) unpack_half<1>(p, me, src, pc, kb0 + 1, nkb, out);
            __syncwarp();                                // every lane has read its row: the buffer is free
            if (PF_NBUF == 1) fetch(u + PF_G, 0);
            if (!(p.debug & 8)) tmem_store32(taddr + 32, out);
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) pf_arrive(pf_smem(&a_full[slot]));
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    } else if (warp == PF_UW) {
        // ------------------------------------------------------------------------------------------ activation copies
        if (lane == 0) {
            const uint8_t *xsrc = reinterpret_cast<const uint8_t *>(p.X16) + (int64_t)blockIdx.y * nkb * PF_B_BYTES;
            bool alive = true;
            for (int kb = 0; kb < nkb && alive; ++kb) {
                const int s = kb % PF_NBS, u = kb / PF_NBS;
                if (u > 0 && (s & 1) == 0) alive = (p.debug & 64) ? pf_wait_poll(pf_smem(&b_empty[s >> 1]), (u - 1) & 1, abort_flag, 24) : pf_wait(pf_smem(&b_empty[s >> 1]), (u - 1) & 1, abort_flag, 24, 20);
                if (!alive) break;
                const uint32_t bar = pf_smem(&b_full[s]);
                if (p.debug & 2) { pf_arrive(bar); continue; }
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"((uint32_t)PF_B_BYTES) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                             :: "r"(pf_smem(smem + s * PF_B_BYTES)), "l"(xsrc + (int64_t)kb * PF_B_BYTES), "r"((uint32_t)PF_B_BYTES), "r"(bar)
                             : "memory");
            }
        }
    } else {
        // ------------------------------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, fp16 x fp16, both operands K-major, N = 256, M = 128
            constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(PF_TOK >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            // descriptors of the activation stages differ only in the start address field: one addition per MMA
            const uint64_t dbase = pf_desc(pf_smem(smem), PF_TOK * 16, 128);
            const uint32_t dlo0 = (uint32_t)dbase, dhi = (uint32_t)(dbase >> 32);
            bool alive = true;
            int s = 0;                                   // activation stage and the parity of its current use
            uint32_t bpar = 0;
            for (int kb = 0; kb < nkb && alive; ++kb) {
                const int unit = kb >> 1, slot = unit & (PF_NU - 1);
                if ((kb & 1) == 0) alive = (p.debug & 64) ? pf_wait_poll(pf_smem(&a_full[slot]), (uint32_t)(unit / PF_NU) & 1u, abort_flag, 25) : pf_wait(pf_smem(&a_full[slot]), (uint32_t)(unit / PF_NU) & 1u, abort_flag, 25, 32);
                if (alive) alive = (p.debug & 64) ? pf_wait_poll(pf_smem(&b_full[s]), bpar, abort_flag, 26) : pf_wait(pf_smem(&b_full[s]), bpar, abort_flag, 26, 32);
                if (!alive) break;
                if ((kb & 1) == 0) asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t a_t = tmem + 256u + (uint32_t)(slot * 64 + (kb & 1) * 32);
                const uint32_t dlo = dlo0 + (uint32_t)(s * (PF_B_BYTES >> 4));
                if (!(p.debug & 16)) {
#pragma unroll
                    for (int kk = 0; kk < PF_BK / 16; ++kk) {
                        // 16 columns of K: 8 columns of tensor memory (two fp16 each) and two 8-column groups of activations
                        uint64_t db;
                        asm volatile("mov.b64 %0, {%1, %2};\n" : "=l"(db) : "r"(dlo + (uint32_t)(kk * ((2 * PF_TOK * 16) >> 4))), "r"(dhi));
                        const uint32_t accumulate = (kb > 0 || kk > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                            " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n}\n"
                            :: "r"(tmem), "r"(a_t + (uint32_t)(8 * kk)), "l"(db), "r"(IDESC), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
                            : "memory");
                    }
                }
                if ((kb & 1) || kb == nkb - 1) {         // a pair of K blocks frees its two activation stages and its weight slot
                    if ((p.debug & 48) == 48) {          // tuning aid, only without MMAs: plain arrivals instead of commits
                        pf_arrive(pf_smem(&b_empty[s >> 1]));
                        pf_arrive(pf_smem(&a_empty[slot]));
                    } else {
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(pf_smem(&b_empty[s >> 1])) : "memory");
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(pf_smem(&a_empty[slot])) : "memory");
                    }
                }
                if (kb == nkb - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(pf_smem(&all_done)) : "memory");
                if (++s == PF_NBS) { s = 0; bpar ^= 1u; }
            }
        }
    }

    // ---- epilogue: tensor memory -> registers -> Y.  A warp reads the 32 lanes (warp & 3) * 32 ...; every group of four
    // warps takes its share of the 256 tokens.
    if (warp < 4 * PF_EG) {
        bool alive = !*abort_flag;
        if (alive) alive = pf_wait(pf_smem(&all_done), 0, abort_flag, 27, 100);
        alive = __all_sync(0xffffffffu, alive);          // tcgen05.ld is warp-wide: all lanes or none
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (alive) {
            const int lq = (warp & 3) * 32;
            const int cbeg = (warp >> 2) * (PF_TOK / PF_EG), cend = cbeg + PF_TOK / PF_EG;
            const int row = me.row;
            const float ts = row >= 0 ? __ldg(p.tau_s + row) : 0.f, ms = row >= 0 ? __ldg(p.min_s + row) : 0.f;
            for (int c0 = cbeg; c0 < cend; c0 += 32) {
                uint32_t d[32];
                const uint32_t taddr = tmem + ((uint32_t)lq << 16) + (uint32_t)c0;
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
    if (*abort_flag && warp == PF_UW) {                      // copies may still be in flight: let them land before the CTA goes
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"((uint32_t)PF_TMEM_COLS) : "memory");
}

// X (M, P) of any input type -> saturated fp16 in the tiled order, tokens padded to Mpad with zeros, and the sums of
// the narrowed values per token and column range (fixed order: a thread sums its groups in order, then eight warps are
// added in order).  With escapes a second, column-major copy (P, Mpad) is written for the escape pass.  Block = 32 tokens (lane) x 8 warps; blockIdx.y = column range.
__global__ void __launch_bounds__(256) prefill_narrow_kernel(const void *__restrict__ X, int x_dtype, int M, int Mpad, int P,
                                                             __half *__restrict__ X16, __half *__restrict__ X16T,
                                                             float *__restrict__ sumx) {
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
        {
            const __half t[8] = {h[0], h[2], h[1], h[3], h[4], h[6], h[5], h[7]};       // see pair_order
            *reinterpret_cast<uint4 *>(X16 + x16_index(n, g * 8, nkb)) = *reinterpret_cast<const uint4 *>(t);
        }
        if (X16T) {                                      // column-major copy for the escape pass: tokens contiguous
#pragma unroll
            for (int k = 0; k < 8; ++k) X16T[(int64_t)(g * 8 + k) * Mpad + n] = h[k];
        }
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

// Y[m, q] += sum over the escapes of row q of x16[m, col] * (exact - band), in stored order.  Block = 32 consecutive
// rows x 256 tokens.  Phase 1: warp w owns rows w, w + 8, w + 16, w + 24; a lane owns eight neighbouring tokens, so an
// escape costs the warp ONE 512-byte read of its column in the column-major copy and eight FMAs per lane.  Phase 2: the
// sums cross shared memory so that a thread owns one token and updates 128 contiguous bytes of Y.
__global__ void __launch_bounds__(256) prefill_escapes_kernel(const int *__restrict__ esc_ptr, const int *__restrict__ esc_col,
                                                              const float *__restrict__ esc_delta, const __half *__restrict__ X16T,
                                                              float *__restrict__ Y, int Q, int M, int Mpad) {
    __shared__ float E[256][33];
    const int q0 = blockIdx.x * 32, n0 = blockIdx.y * 256;
    const int qe = min(Q, q0 + 32);
    if (__ldg(esc_ptr + q0) == __ldg(esc_ptr + qe)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4 *xt = reinterpret_cast<const uint4 *>(X16T + n0 + 8 * lane);       // Mpad is a multiple of 256
    const int64_t ld = Mpad >> 3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int q = q0 + warp + 8 * j;
        float acc[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) acc[t] = 0.f;
        if (q < Q) {
            const int e0 = __ldg(esc_ptr + q), e1 = __ldg(esc_ptr + q + 1);
            for (int e = e0; e < e1; e += 2) {           // two at a time: the loads overlap
                const int ee = min(e + 1, e1 - 1);
                const float d0 = __ldg(esc_delta + e), d1 = e + 1 < e1 ? __ldg(esc_delta + ee) : 0.f;
                const uint4 v0 = __ldg(xt + (int64_t)__ldg(esc_col + e) * ld), v1 = __ldg(xt + (int64_t)__ldg(esc_col + ee) * ld);
                const __half2 *h0 = reinterpret_cast<const __half2 *>(&v0), *h1 = reinterpret_cast<const __half2 *>(&v1);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float2 f = __half22float2(h0[t]);
                    acc[2 * t] = __fmaf_rn(f.x, d0, acc[2 * t]);
                    acc[2 * t + 1] = __fmaf_rn(f.y, d0, acc[2 * t + 1]);
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float2 f = __half22float2(h1[t]);
                    acc[2 * t] = __fmaf_rn(f.x, d1, acc[2 * t]);
                    acc[2 * t + 1] = __fmaf_rn(f.y, d1, acc[2 * t + 1]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) E[8 * lane + t][warp + 8 * j] = acc[t];
    }
    __syncthreads();
    const int n = n0 + threadIdx.x;
    if (n >= M) return;
    float *y = Y + (int64_t)n * Q + q0;
    const float *er = E[threadIdx.x];
    if ((Q & 3) == 0 && q0 + 32 <= Q) {
#pragma unroll
        for (int r = 0; r < 32; r += 4) {
            float4 v = *reinterpret_cast<float4 *>(y + r);
            v.x += er[r]; v.y += er[r + 1]; v.z += er[r + 2]; v.w += er[r + 3];
            *reinterpret_cast<float4 *>(y + r) = v;
        }
    } else {
        for (int r = 0; r < 32; ++r)
            if (q0 + r < Q) y[r] += er[r];
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

static int g_prefill_debug = 0;

static int launch_prefill(const PrefillParams &prm, cudaStream_t st) {
    static thread_local int granted_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != granted_dev) {
        if (cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM) != cudaSuccess)
            return cuda_status("qvb8_prefill: shared memory opt-in");
        granted_dev = dev;
    }
    const int slots = prm.max_tiles * 16;
    const dim3 grid((unsigned)((slots + 127) / 128), (unsigned)(prm.Mpad / PF_TOK));
    prefill_kernel<<<grid, PF_THREADS, PF_SMEM, st>>>(prm);
    return cuda_status("qvb8_prefill");
}

}  // namespace qv

QV_API void qvb8_prefill_set_tuning(int debug) { qv::g_prefill_debug = debug; }

QV_API int64_t qvb8_prefill_scratch_bytes(int64_t M, int64_t Q, int64_t P) {
    if (M <= 0 || P <= 0 || Q < 0) return 0;
    const int64_t Mpad = (M + qv::PF_TOK - 1) / qv::PF_TOK * qv::PF_TOK;
    return 2 * qv::up256(Mpad * P * 2) + qv::up256(qv::PF_KS * Mpad * 4) + qv::up256((Q + 1) * 4);
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
    if (w->ids_bytes >= (1ll << 32)) return fail(QVB8_ERR_ARG, "qvb8_prefill: packs of 4 GiB and more are not supported");
    if (!plan || !aligned(plan, 256)) return fail(QVB8_ERR_ARG, "qvb8_prefill: the pack's plan is needed (qvb8_plan_build), 256-byte aligned");
    const int64_t need = qvb8_prefill_scratch_bytes(M, w->Q, w->P);
    if (!scratch || scratch_bytes < need || !aligned(scratch, 256))
        return fail(QVB8_ERR_SCRATCH, "qvb8_prefill: scratch of %lld bytes (256-byte aligned) needed, %lld given", (long long)need, (long long)scratch_bytes);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int64_t Mpad = (M + PF_TOK - 1) / PF_TOK * PF_TOK;
    uint8_t *sc = reinterpret_cast<uint8_t *>(scratch);
    __half *X16 = reinterpret_cast<__half *>(sc);
    __half *X16T = reinterpret_cast<__half *>(sc + up256(Mpad * w->P * 2));      // written only for packs with escapes
    float *sumx = reinterpret_cast<float *>(sc + 2 * up256(Mpad * w->P * 2));
    int *wide = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(sumx) + up256(PF_KS * Mpad * 4));      // [0] count, then rows
    prefill_narrow_kernel<<<dim3((unsigned)(Mpad / 32), PF_KS), 256, 0, st>>>(X, x_dtype, (int)M, (int)Mpad, (int)w->P, X16, w->n_esc > 0 ? X16T : nullptr, sumx);
    if (int rc = cuda_status("qvb8_prefill narrow")) return rc;

    const PlanLayout L = plan_layout(w->Q, w->n_esc);
    const uint8_t *pb = reinterpret_cast<const uint8_t *>(plan);
    PrefillParams prm{w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, reinterpret_cast<const TileDesc *>(pb + L.tiles), L.max_tiles,
                      X16, sumx, Y, (int)w->Q, (int)w->P, (int)M, (int)Mpad, g_prefill_debug};
    if (int rc = launch_prefill(prm, st)) return rc;

    if (cudaMemsetAsync(wide, 0, sizeof(int), st) != cudaSuccess) return cuda_status("qvb8_prefill memset");
    prefill_wide_list_kernel<<<(unsigned)((w->Q + 255) / 256), 256, 0, st>>>(w->nbits, (int)w->Q, wide + 1, wide);
    prefill_wide_rows_kernel<<<dim3(64, (unsigned)((M + 7) / 8)), 256, 0, st>>>(prm, wide + 1, wide);
    if (int rc = cuda_status("qvb8_prefill wide rows")) return rc;
    if (w->n_esc > 0) {
        prefill_escapes_kernel<<<dim3((unsigned)((w->Q + 31) / 32), (unsigned)(Mpad / 256)), 256, 0, st>>>(
            reinterpret_cast<const int *>(pb + L.esc_ptr), reinterpret_cast<const int *>(pb + L.esc_col),
            reinterpret_cast<const float *>(pb + L.esc_delta), X16T, Y, (int)w->Q, (int)M, (int)Mpad);
        if (int rc = cuda_status("qvb8_prefill escapes")) return rc;
    }
    return QVB8_OK;
}
