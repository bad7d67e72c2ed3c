// QVB8 small-M fused decode-in-matmul for sm_100a:  Y[m, q] = sum_c X[m, c] * W[q, c],  1 <= M <= 48,
// W read ONCE from HBM as bit-packed ids and never materialised.
//
// Replaces the reference's GEMV family and its mma.sync verify kernel
// (formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:306-453 qvb8_gemv_multi_v3, :463-489 split-K, :507-533 escape
// correction, :1813-2441 qvb8_mma_*), and the per-module row ordering the reference computes for it
// (formats/qvb8/module.py:230-288 _mma_order / _esc_row_starts).
//
// Arithmetic.  With w = min_s + id * tau_s the row sum factors (the identity the reference states at
// qvb8_cuda.cu:3-9):   y[m, q] = min_s[q] * sum_c x[m, c]  +  tau_s[q] * sum_c x[m, c] * id[q, c].
// The ids are small integers, exact in fp16, so the inner sum runs on the tensor cores (fp16 x fp16 -> fp32,
// products exact, fp32 accumulation) and the per-weight CUDA-core work is only the bit extraction.  The weight
// is therefore the un-narrowed band value, the contract of the reference's M <= 8 GEMV; X is narrowed to saturated
// fp16 first, as every fp16-mode path of the reference does (:761-841).
//
// Plan.  Rows of a pack have different widths.  Once per pack, qvb8_plan_build sorts the rows by width (stable) into
// 16-row TILES of one width and writes one 400-byte descriptor per tile (rows, byte offsets, origins, steps, escape
// ranges), and regroups the escapes by row with the difference (exact - band) precomputed.  The product kernel only
// follows descriptors.
//
// Roofline: HBM.  Per weight the kernel moves nbits/8 bytes (about 0.8).  What HBM sees matters as much as how
// much: a row is a contiguous byte range, so for each of the 16 rows of a tile a producer warp fetches ONE
// contiguous run of columns per stage with a bulk asynchronous copy (cp.async.bulk with an evict-first L2 hint,
// completion counted on an mbarrier), several stages ahead; the tile's descriptor travels with its first stage.
// CTAs are persistent and hold up to four independent PIPES (producer warp + four consumer warps + finishing warp
// each, own rings and barriers), so a stall in one pipe's hand-over does not idle the SM's copy stream.
//
// Math.  Four consumer warps each take one 128-column chunk of the stage.  Thread (g = lane / 4, t = lane % 4) owns
// the 32 ids of rows g and g + 8 that start at column 32 t -- exactly nb 32-bit words -- and turns them into the A
// fragments of eight m16n8k16 MMAs.  Two ids are converted per instruction: a funnel shift puts one id in the low
// half-word and one in the high half-word of a register, `(r & mask) | 0x64006400` makes the two fp16 numbers
// 1024 + id * 2^e, and one HFMA2 removes the 1024 and the 2^e exactly.  At the end of a tile the warps hand their
// partial accumulators to the pipe's finishing warp through a double-buffered area of shared memory and go on
// streaming; the finishing warp adds them in warp order, applies min_s / tau_s and the per-token sum of X (collected
// while X was staged), adds the escape corrections, and writes the result.  K-ranges of one tile are added in range
// order by whichever CTA finishes the tile last (a ticket counter per tile).
//
// Lists.  One launch can run up to 128 independent products (qvb8_small_m_group): the job table travels by value in
// the kernel's parameters.  All (tile, stage) units of the list form ONE sequence that is cut into equal contiguous
// per-CTA ranges, so a CTA meets one or two jobs per launch and its rings never drain at a job boundary; at a
// boundary the consumer warps restage X for the next job from global memory while the producer is already copying
// that job's first stages.  Rarely executed serial work is expensive on an SM whose other warps stream (a dependent
// chain costs on the order of 100 cycles per instruction there), so for lists the escape corrections run in a
// pre-pass kernel, one thread per (tile, row), that writes them into Y; the streaming kernel then adds its result
// to Y with one atomic add per element -- one writer per element after the ticket, so the sum order stays fixed.
//
// Every sum has a fixed order: results are identical from run to run.  A list agrees with separate calls to fp32
// rounding (the grouping of the K partial sums differs), not bit for bit.
//
// Waits.  Every wait on an mbarrier is bounded: after two seconds (or SPIN_LIMIT polls) the waiter raises a per-CTA
// abort flag and a device-wide error word (qvb8_device_status), every other waiter gives up too, and the kernel
// runs to its end with a meaningless result instead of hanging.
#include "common.cuh"
#include "plan.cuh"

#include <mutex>

namespace qv {

int launch_fix_escapes(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y, cudaStream_t st);
int launch_small_m_generic(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y,
                           cudaStream_t st);
int check_small_m_args(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, const float *Y,
                       const char *who);
int prefill_error_word(int *out);                 // qvb8_prefill.cu
int peer_error_word(int *out);                    // qvb8_peer.cu
int peer_error_reset();

constexpr int KC = 128;                   // columns per chunk
constexpr int NW = 4;                     // consumer warps
constexpr int MAX_CPS = 16;               // most chunks per stage (a stage holds cps chunks, cps a multiple of NW)
constexpr int PRODUCER_WARP = NW;         // issues the bulk copies
constexpr int FINISHER_WARP = NW + 1;     // escape corrections, cross-warp sums, scaling, output
constexpr int PIPE_THREADS = (NW + 2) * 32;  // threads of one pipe
constexpr int MAX_STAGES = 6;
constexpr int MAX_PIPES = 4;               // pipes per CTA at most
#ifndef QVB8_PIPES_NT1
#define QVB8_PIPES_NT1 4
#endif
constexpr int PIPES_NT1 = QVB8_PIPES_NT1;  // pipes per CTA for up to 8 tokens
constexpr int XCH_SLOTS = (MAX_PIPES - 1) * (MAX_PIPES - 1);   // [owner pipe][contributor]
constexpr int64_t TICKET_BYTES = 256 * 1024;  // fixed-size counter area at the START of the scratch (one counter per
                                              // tile), so that calls of different sizes sharing one scratch never
                                              // find partial sums in it
constexpr int MAX_TICKET_TILES = (int)(TICKET_BYTES / 4);
constexpr int MAX_M = 48;
constexpr int SPIN_LIMIT = 1 << 22;

__device__ int g_error_word = 0;          // first timeout of any kernel of this library (0 = none)
__device__ unsigned long long g_trace[32];   // tuning aid: nanosecond stamps of CTA (0, 0) when debug bit 1 is set
__device__ __forceinline__ void trace(int debug, int slot) {
    if ((debug & 2) && blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_trace[slot] = t;
    }
}

constexpr int DESC_SLOT = 416;            // descriptor area of a side slot
constexpr int ESC_CAP_MIN = 64, ESC_CAP_MAX = 512;   // escape entries that travel with a descriptor (a launch picks the
                                                     // capacity from its widest job; the rest is read from global memory)
constexpr int NSIDE = 3;                  // side slots per pipe: descriptors and escapes of the visits ahead
__host__ __device__ constexpr int64_t side_slot_bytes(int esc_cap) { return DESC_SLOT + (int64_t)esc_cap * 8; }
// Entry capacity for rows of P columns: what 16 rows hold at 1.5 escapes per thousand weights (packs made with the
// outliers escaped carry about 1 per thousand), within the limits above.
__host__ __device__ constexpr int esc_cap_for(int64_t P) {
    const int64_t want = (16 * P * 3 / 2000 + 31) / 32 * 32;
    return (int)(want < ESC_CAP_MIN ? ESC_CAP_MIN : want > ESC_CAP_MAX ? ESC_CAP_MAX : want);
}

// Bytes of a pipe's escape area: the finishing warp's corrections [16][M] and, for one token, a staging array of
// (difference, activation) pairs of the tile's entries (see the finishing warp).
__host__ __device__ constexpr int64_t corr_stride_bytes(int64_t M) { return (16 * M * 4 + 127) / 128 * 128; }
constexpr int INLINE_ESC_MAX_M = 4;       // lists of up to this many tokens sum their escapes on the consumer warps
__host__ __device__ constexpr int64_t corr_buffers(int64_t M) { return M <= INLINE_ESC_MAX_M ? 2 * NW : 2; }
__host__ __device__ constexpr int64_t corr_bytes(int64_t M, int esc_cap) {
    // [16][M] buffers: a single launch's finishing warp uses the first; a list's consumer warps write one each per visit,
    // two sets alternating like the hand-over buffers ([2][NW][16][M]); then the one-token staging array
    return corr_buffers(M) * corr_stride_bytes(M) + (M == 1 ? (int64_t)esc_cap * 8 : 0);
}

// Per-CTA control block in static shared memory.
struct PipeControl {
    alignas(8) uint64_t full[MAX_STAGES];
    alignas(8) uint64_t empty[MAX_STAGES];
    alignas(8) uint64_t side_full[NSIDE];   // a visit's descriptor and escapes have landed
    alignas(8) uint64_t side_empty[NSIDE];  // ... and the four consumer warps and the finishing warp are done with them
    alignas(8) uint64_t red_full[2];      // the consumer warps' partial sums of a visit are in hand-over buffer b
    alignas(8) uint64_t red_empty[2];     // ... and have been taken by the finishing warp
};
struct Control {
    uint32_t amax[MAX_M];                 // x_mode 1: bits of the largest |x| of a token in this K-range
    uint8_t kexp[MAX_M];                  // x_mode 1: token m is staged as x * 2^-kexp[m] and its results multiplied back
    int abort;
    alignas(16) uint32_t pair_table[24];  // pair-conversion constants of widths 3..8 (see pair_const)
    alignas(8) uint64_t amax_ready;       // x_mode 1: every consumer warp has folded its share into amax
    alignas(8) uint64_t x_ready;          // once per job: every consumer warp has staged its slice of the activations
    alignas(8) uint64_t job_done;         // once per job boundary: every consumer warp has left the job before
    alignas(8) uint64_t fin_started;      // once per job: every finishing warp has reached the job and taken its activation sums
    alignas(8) uint64_t xch_full[XCH_SLOTS];   // [owner pipe][contributor]: a contributed part of a shared tile is in place
    alignas(8) uint64_t xch_empty[XCH_SLOTS];  // ... and the owner has taken it
    PipeControl pipe[MAX_PIPES];
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier / bulk copy ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// One poll.  The barrier unit parks the warp until the phase completes or the time hint (nanoseconds) runs out, so a
// waiting warp issues a handful of instructions per hint period instead of competing with the working warps.
constexpr uint32_t WAIT_HINT_NS = 20000;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;      // a wait gives up after two seconds (or SPIN_LIMIT polls)
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(WAIT_HINT_NS) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false if the barrier did not complete (this waiter or another one gave up).
// backoff_ns > 0: the waiter is not on the critical path (a producer waiting for a free slot, a finishing warp waiting
// for sums) and sleeps between polls, leaving the issue slots to the warps that compute.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code,
                                            uint32_t backoff_ns) {
    const uint64_t t0 = global_ns();
    for (int i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (backoff_ns) __nanosleep(backoff_ns);
        if ((i & 7) == 7) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > WAIT_LIMIT_NS) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_error_word, 0, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code,
                                          uint32_t backoff_ns = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, code, backoff_ns);
}
// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned); completion is counted
// on `bar`.  The destination is this CTA's own shared memory.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// The same copy marked evict-first in L2: the packed weights are read once per product, and a launch streams far more of
// them than the L2 holds.  Without the hint they push everything else out -- the kernel's own instructions, tile
// descriptors, activations -- and whatever then misses in L2 queues behind the weight stream in a saturated HBM
// (microseconds per miss: a rarely executed code path then costs more than the tile it finishes).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_stream(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
}

// Programmatic dependent launch: everything before pdl_wait() may overlap the tail of the previous kernel in the
// stream (it must not touch memory that kernel writes); both are no-ops for a normal launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Pairing of a width: ids f and f + D share a register.  E > 0: the low id sits at mantissa bit E and the high id at
// bit 0 of the upper half-word; E < 0: the low id at bit 0, the high id at mantissa bit -E.  (nb * D == 16 - E.)
template <int NB> struct Pairing;
template <> struct Pairing<8> { static constexpr int D = 2, E = 0; };
template <> struct Pairing<7> { static constexpr int D = 2, E = 2; };
template <> struct Pairing<6> { static constexpr int D = 2, E = 4; };
template <> struct Pairing<5> { static constexpr int D = 4, E = -4; };
template <> struct Pairing<4> { static constexpr int D = 4, E = 0; };
template <> struct Pairing<3> { static constexpr int D = 4, E = 4; };

// fp16 bit patterns of 2^-e and -1024 * 2^-e (written as integers: the conversion intrinsics are opaque to constant
// folding and would run on the conversion pipe for every pair).
__host__ __device__ constexpr uint32_t h_pow2(int e) { return (uint32_t)(15 - e) << 10; }
__host__ __device__ constexpr uint32_t h_neg1024_pow2(int e) { return 0x8000u | ((uint32_t)(25 - e) << 10); }

// The four constants of a width, held in registers for a whole tile.  They are read from a small table in shared
// memory with volatile loads: values the compiler can see (literals, or moves of literals) it re-creates next to
// every use -- one extra instruction per pair, measured -- because the fp16 multiply-add takes only one of its two
// constants as an immediate.
struct PairConst { uint32_t mask, magic, scale, bias; };
__host__ __device__ constexpr uint32_t pair_const_word(int nb, int k) {
    const int D = nb >= 6 ? 2 : 4;
    const int E = 16 - nb * D;                                   // Pairing<nb>::E
    const int EL = E > 0 ? E : 0, EH = E < 0 ? -E : 0;
    const uint32_t FM = (1u << nb) - 1u;
    return k == 0 ? ((FM << EL) | (FM << (16 + EH)))
         : k == 1 ? 0x64006400u
         : k == 2 ? (h_pow2(EL) | (h_pow2(EH) << 16))
                  : (h_neg1024_pow2(EL) | (h_neg1024_pow2(EH) << 16));
}
constexpr int PAIR_TABLE_WORDS = 6 * 4;                          // widths 3..8
__device__ __forceinline__ PairConst pair_const(const uint32_t *table, int nb) {
    const uint32_t a = smem_u32(table + (nb - 3) * 4);
    PairConst c;
    asm volatile("ld.volatile.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(c.mask), "=r"(c.magic), "=r"(c.scale), "=r"(c.bias) : "r"(a));
    return c;
}

// Register holding fp16(id[fa]) in the low half and fp16(id[fa + D]) in the high half, from the nb words W of a
// thread's 32-id block.  All shifts fold to constants after unrolling.
template <int NB>
__device__ __forceinline__ uint32_t pair_reg(const uint32_t (&W)[NB], int fa, const PairConst &pc) {
    constexpr int D = Pairing<NB>::D, E = Pairing<NB>::E;
    constexpr int EL = E > 0 ? E : 0;            // mantissa shift of the low id
    constexpr int EH = E < 0 ? -E : 0;           // mantissa shift of the high id
    static_assert(NB * D == 16 + EH - EL, "pairing does not line the two ids up");
    static_assert(EL + NB <= 10 && EH + NB <= 10, "id does not fit the fp16 mantissa");
    const int s = NB * fa - EL;                  // bit of the block that must land on bit 0
    uint32_t r;
    if (s < 0) {
        r = W[0] << (-s);
    } else {
        const int wi = s >> 5, sh = s & 31;
        const int top = sh + 16 + EH + NB;       // one past the highest bit needed, relative to W[wi]
        if (sh == 0) r = W[wi];
        else if (top <= 32) r = W[wi] >> sh;
        else asm("shf.r.wrap.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(W[wi]), "r"(W[wi + 1 < NB ? wi + 1 : wi]), "r"(sh));
    }
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(r), "r"(pc.mask), "r"(pc.magic));   // (r & mask) | magic:
    if constexpr (EL == 0 && EH == 0) {                                                         // 1024 + id * 2^shift, twice
        asm("sub.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(r), "r"(pc.magic));
    } else {
        asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(r), "r"(pc.scale), "r"(pc.bias));
    }
    return r;
}

// The nb words of a thread's block, with the widest conflict-free shared-memory loads for that width.
template <int NB>
__device__ __forceinline__ void load_block(uint32_t addr, uint32_t (&W)[NB]) {
    if constexpr (NB == 8) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(W[0]), "=r"(W[1]), "=r"(W[2]), "=r"(W[3]) : "r"(addr));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+16];\n" : "=r"(W[4]), "=r"(W[5]), "=r"(W[6]), "=r"(W[7]) : "r"(addr));
    } else if constexpr (NB == 4) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(W[0]), "=r"(W[1]), "=r"(W[2]), "=r"(W[3]) : "r"(addr));
    } else if constexpr (NB == 6) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(W[0]), "=r"(W[1]) : "r"(addr));
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+8];\n" : "=r"(W[2]), "=r"(W[3]) : "r"(addr));
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+16];\n" : "=r"(W[4]), "=r"(W[5]) : "r"(addr));
    } else {
        static_assert(NB == 8 || NB == 4 || NB == 6, "odd widths are specialised below");
    }
}
// odd widths: nb scalar loads (an odd stride in words spreads the 32 lanes over all banks)
template <>
__device__ __forceinline__ void load_block<7>(uint32_t addr, uint32_t (&W)[7]) {
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(W[0]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+4];\n" : "=r"(W[1]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+8];\n" : "=r"(W[2]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+12];\n" : "=r"(W[3]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+16];\n" : "=r"(W[4]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+20];\n" : "=r"(W[5]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+24];\n" : "=r"(W[6]) : "r"(addr));
}
template <>
__device__ __forceinline__ void load_block<5>(uint32_t addr, uint32_t (&W)[5]) {
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(W[0]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+4];\n" : "=r"(W[1]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+8];\n" : "=r"(W[2]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+12];\n" : "=r"(W[3]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+16];\n" : "=r"(W[4]) : "r"(addr));
}
template <>
__device__ __forceinline__ void load_block<3>(uint32_t addr, uint32_t (&W)[3]) {
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(W[0]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+4];\n" : "=r"(W[1]) : "r"(addr));
    asm volatile("ld.shared.u32 %0, [%1+8];\n" : "=r"(W[2]) : "r"(addr));
}

// Bytes between rows of a stage.  The chunks of a row lie back to back (one contiguous copy per row and stage); the
// stride adds padding so that the 32 lanes of a warp, which read rows g and columns 32 t of ONE chunk, fall on
// distinct banks.
__host__ __device__ constexpr bool stride_ok(int nb, int rs) {
    return nb == 8 ? (rs / 16) % 8 == 1                  // 16-byte loads, quarter warps (rows 2i, 2i+1)
         : nb == 4 ? (rs / 16) % 8 == 4
         : nb == 6 ? (rs / 8) % 16 == 12                 // 8-byte loads, half warps (rows 4i .. 4i+3)
                   : (rs / 4) % 32 == (4 * nb) % 32;     // 4-byte loads, whole warp
}
__host__ __device__ constexpr int stage_row_stride(int nb, int cps) {
    int rs = 16 * nb * cps;
    while (!stride_ok(nb, rs)) rs += 16;
    return rs;
}

// One 128-column chunk of a 16-row tile of width NB: 8 MMAs per token group.
//   wa, wb   shared addresses of this thread's blocks in rows g and g + 8 of the stage
//   xa       shared address of this thread's first activation slot of the chunk (token 8n + g -> + n * 512 bytes)
//   xstep    bytes between the slots of consecutive 8-column groups (= 4 * MP * 16; 0 for lanes without a token)
//   DUAL     true: a second activation layout exists for widths that pair ids at distance 4 (xa points into it);
//            false: only layout A is staged and those widths rebuild their operands with byte permutes
template <int NB, int NT, bool DUAL>
__device__ __forceinline__ void chunk_mma(uint32_t wa, uint32_t wb, uint32_t xa, uint32_t xstep, float (&acc)[NT][4],
                                          const PairConst &pc) {
    constexpr int D = Pairing<NB>::D;
    uint32_t Wa[NB], Wb[NB];
    load_block<NB>(wa, Wa);
    load_block<NB>(wb, Wb);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // activations of columns 32 t + 8 i .. + 7 for this thread's token(s), already in fragment order:
        // words (2h, 2h + 1) are the B operands of MMA h of this group
        uint32_t xw[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(xw[n][0]), "=r"(xw[n][1]), "=r"(xw[n][2]), "=r"(xw[n][3])
                         : "r"(xa + i * xstep + n * 512));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // ids of this MMA: D == 2 -> {8i+4h .. 8i+4h+3} paired (f, f+2);  D == 4 -> {8i+2h, +1, +4, +5} paired (f, f+4)
            const int f0 = D == 2 ? 8 * i + 4 * h : 8 * i + 2 * h;
            const uint32_t a0 = pair_reg<NB>(Wa, f0, pc), a2 = pair_reg<NB>(Wa, f0 + 1, pc);
            const uint32_t a1 = pair_reg<NB>(Wb, f0, pc), a3 = pair_reg<NB>(Wb, f0 + 1, pc);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                if constexpr (D == 2 || DUAL) {
                    mma16816(acc[n], a0, a1, a2, a3, xw[n][2 * h], xw[n][2 * h + 1]);
                } else {
                    // layout A words are (x0 x2)(x1 x3)(x4 x6)(x5 x7); distance-4 pairs are (x[2h] x[2h+4]), (x[2h+1] x[2h+5])
                    const uint32_t sel = h == 0 ? 0x5410u : 0x7632u;
                    mma16816(acc[n], a0, a1, a2, a3, __byte_perm(xw[n][0], xw[n][2], sel),
                             __byte_perm(xw[n][1], xw[n][3], sel));
                }
            }
        }
    }
}

// Activation layouts in shared memory.  A 16-byte slot holds the 8 activations of one token for one 8-column group;
// slots are ordered (chunk, group-in-block i, token, block t): lane (g, t) of a warp reads token g, block t, so the 32
// lanes of a 16-byte load read 512 consecutive bytes in lane order and no two lanes of a quarter-warp share a bank
// (with the block outside the token, lanes of equal g lay 128 bytes apart: four-way conflicts on every such load).  Inside a slot the halves are permuted so that word
// pairs are the B operands directly:  layout A (ids paired at distance 2): x0 x2 x1 x3 x4 x6 x5 x7;
// layout B (distance 4): x0 x4 x1 x5 x2 x6 x3 x7.
__device__ __forceinline__ int slot_of(int c, int m, int MP) {
    const int chunk = c >> 7, t = (c >> 5) & 3, i = (c >> 3) & 3;
    return ((chunk * 4 + i) * MP + m) * 4 + t;
}
__device__ __forceinline__ int pos_a(int e) { return (e & 4) | ((e & 1) << 1) | ((e >> 1) & 1); }
// natural-order read of X[m, c] (c relative to the CTA's first column) from layout A
__device__ __forceinline__ float xs_read(const __half *xs, int c, int m, int MP) {
    return __half2float(xs[(slot_of(c, m, MP) << 3) + pos_a(c & 7)]);
}

// 16 bytes from global memory through the read-only path, or (GLOBAL = false) from wherever a generic pointer leads
template <bool GLOBAL>
__device__ __forceinline__ uint4 load16(const void *ptr) {
    if constexpr (GLOBAL) return __ldg(reinterpret_cast<const uint4 *>(ptr));
    else return *reinterpret_cast<const uint4 *>(ptr);
}
template <int XT, bool GLOBAL>
__device__ __forceinline__ void stage_x8(const void *__restrict__ X, int64_t off, uint32_t (&h)[8], float sc) {
    // h[k] = fp16 bits of the k-th activation times sc (1, or a token's power-of-two prescale), saturated
    if constexpr (XT == QVB8_F16) {
        const uint4 u = load16<GLOBAL>(reinterpret_cast<const __half *>(X) + off);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { h[2 * k] = w[k] & 0xffffu; h[2 * k + 1] = w[k] >> 16; }
    } else if constexpr (XT == QVB8_BF16) {
        const uint4 u = load16<GLOBAL>(reinterpret_cast<const __nv_bfloat16 *>(X) + off);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            h[2 * k] = __half_as_ushort(sat_half(__uint_as_float(w[k] << 16) * sc));
            h[2 * k + 1] = __half_as_ushort(sat_half(__uint_as_float(w[k] & 0xffff0000u) * sc));
        }
    } else {
        const uint4 a = load16<GLOBAL>(reinterpret_cast<const float *>(X) + off);
        const uint4 b = load16<GLOBAL>(reinterpret_cast<const float *>(X) + off + 4);
        const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) h[k] = __half_as_ushort(sat_half(__uint_as_float(v[k]) * sc));
    }
}

// Largest |x| of 8 activations as float bits (NaN and infinity count as the largest finite exponent and above:
// their staging saturates anyway).  fp16 input never needs a prescale.
template <int XT>
__device__ __forceinline__ uint32_t amax_x8(const void *__restrict__ X, int64_t off) {
    uint32_t mx = 0u;
    if constexpr (XT == QVB8_BF16) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(X) + off));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { mx = max(mx, (w[k] << 16) & 0x7fffffffu); mx = max(mx, w[k] & 0x7fff0000u); }
    } else if constexpr (XT == QVB8_F32) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(X) + off));
        const uint4 b = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(X) + off) + 1);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) mx = max(mx, w[k] & 0x7fffffffu);
    }
    return mx;
}
// Prescale exponent of a token whose largest magnitude has these float bits: the smallest k >= 0 that brings it below
// 2^16 (fp16 holds up to 65504; the narrowing still saturates the sliver between).
__device__ __forceinline__ int prescale_exp(uint32_t amax_bits) {
    const int e = (int)(amax_bits >> 23) - 127;
    return e > 15 ? min(e - 15, 112) : 0;
}
__device__ __forceinline__ float pow2f(int k) { return __uint_as_float((uint32_t)(127 + k) << 23); }

// ---------------------------------------------------------------------------------------------------------------
// plan build (once per pack)

__device__ __forceinline__ int row_class(int nb, int64_t bit_off) {
    return (nb >= 3 && nb <= 8 && (bit_off & 127) == 0) ? nb - 3 : NCLASS - 1;      // fragment path needs 16-byte aligned rows
}

// Escapes regrouped by row: first escape of every row, column and (exact - band) of every escape.
__global__ void __launch_bounds__(256) escape_plan_kernel(const uint8_t *__restrict__ ids, const float *__restrict__ min_s,
                                                          const float *__restrict__ tau_s,
                                                          const uint8_t *__restrict__ nbits,
                                                          const int64_t *__restrict__ bit_off,
                                                          const int64_t *__restrict__ esc_idx,
                                                          const float *__restrict__ esc_vals, int64_t n_esc, int Q, int P,
                                                          int *__restrict__ esc_ptr, int *__restrict__ esc_col,
                                                          float *__restrict__ esc_delta) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_esc) {
        // a position outside the weight (a corrupt escape list) is clamped to the last row and contributes nothing
        const int64_t f = __ldg(esc_idx + i);
        const bool inside = f >= 0 && f < (int64_t)Q * P;
        const int q = inside ? (int)(f / P) : Q - 1, c = inside ? (int)(f - (int64_t)q * P) : 0;
        const int nb = __ldg(nbits + q);
        const float b = band(field_bytes(ids, __ldg(bit_off + q) + (int64_t)c * nb, nb), __ldg(tau_s + q), __ldg(min_s + q));
        esc_col[i] = c;
        esc_delta[i] = inside ? __ldg(esc_vals + i) - b : 0.f;
        // esc_idx ascends: this escape opens every row after the previous escape's row, up to its own
        int qprev = -1;
        if (i > 0) {
            const int64_t fp = __ldg(esc_idx + i - 1);
            qprev = (fp >= 0 && fp < (int64_t)Q * P) ? (int)(fp / P) : Q - 1;
        }
        for (int r = qprev + 1; r <= q; ++r) esc_ptr[r] = (int)i;
        if (i == n_esc - 1)
            for (int r = q + 1; r <= Q; ++r) esc_ptr[r] = (int)n_esc;
    } else if (i == 0 && n_esc == 0) {
        for (int r = 0; r <= Q; ++r) esc_ptr[r] = 0;
    }
}


// Rows sorted by class (stable) into tiles.  One block: the sort is a counting sort over at most seven classes.
__global__ void __launch_bounds__(1024) plan_tiles_kernel(const uint8_t *__restrict__ nbits,
                                                          const int64_t *__restrict__ bit_off,
                                                          const float *__restrict__ min_s, const float *__restrict__ tau_s,
                                                          const int *__restrict__ esc_ptr, int Q, int max_tiles,
                                                          TileDesc *__restrict__ tiles, int *__restrict__ header) {
    __shared__ int cnt[NCLASS], base_tile[NCLASS], running[NCLASS];
    __shared__ int wtot[32][NCLASS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < NCLASS) { cnt[tid] = 0; running[tid] = 0; }
    __syncthreads();
    {
        int local[NCLASS];
#pragma unroll
        for (int c = 0; c < NCLASS; ++c) local[c] = 0;
        for (int q = tid; q < Q; q += 1024) {
            const int c = row_class(__ldg(nbits + q), __ldg(bit_off + q));
#pragma unroll
            for (int k = 0; k < NCLASS; ++k) local[k] += (c == k);
        }
#pragma unroll
        for (int c = 0; c < NCLASS; ++c)
            if (local[c]) atomicAdd(&cnt[c], local[c]);
    }
    __syncthreads();
    if (tid == 0) {
        int t = 0;
        for (int c = 0; c < NCLASS; ++c) { base_tile[c] = t; t += (cnt[c] + 15) / 16; }
        header[0] = t;
    }
    __syncthreads();
    for (int q0 = 0; q0 < Q; q0 += 1024) {
        const int q = q0 + tid;
        int c = -1, nb = 0;
        int64_t bo = 0;
        if (q < Q) { nb = __ldg(nbits + q); bo = __ldg(bit_off + q); c = row_class(nb, bo); }
        int before = 0;                                     // rows of my class earlier in my warp
#pragma unroll
        for (int k = 0; k < NCLASS; ++k) {
            const uint32_t mk = __ballot_sync(0xffffffffu, c == k);
            if (c == k) before = __popc(mk & ((1u << lane) - 1u));
            if (lane == 0) wtot[warp][k] = __popc(mk);
        }
        __syncthreads();
        if (c >= 0) {
            int pos = running[c] + before;
            for (int w = 0; w < warp; ++w) pos += wtot[w][c];
            TileDesc &d = tiles[base_tile[c] + (pos >> 4)];
            const int s = pos & 15;
            d.row[s] = q;
            d.b16[s] = (uint32_t)(bo >> 7);
            d.ms[s] = __ldg(min_s + q);
            d.ts[s] = __ldg(tau_s + q);
            d.e0[s] = esc_ptr ? __ldg(esc_ptr + q) : 0;
            d.e1[s] = esc_ptr ? __ldg(esc_ptr + q + 1) : 0;
        }
        __syncthreads();
        if (tid < NCLASS) {
            int t = 0;
            for (int w = 0; w < 32; ++w) t += wtot[w][tid];
            running[tid] += t;
        }
        __syncthreads();
    }
    const int ntiles = header[0];
    for (int t = tid; t < ntiles; t += 1024) {
        int c = 0;
        for (int k = 0; k < NCLASS; ++k)
            if (cnt[k] > 0 && t >= base_tile[k] && t < base_tile[k] + (cnt[k] + 15) / 16) c = k;
        const int n = min(16, cnt[c] - 16 * (t - base_tile[c]));
        tiles[t].nb = c == NCLASS - 1 ? 0 : c + 3;
        tiles[t].cnt = n;
        for (int s = n; s < 16; ++s) tiles[t].row[s] = -1;
    }
    // the table is as long as the largest tile count a pack of Q rows can have; the surplus tiles are empty
    for (int t = ntiles + tid; t < max_tiles; t += 1024) {
        tiles[t].nb = 0;
        tiles[t].cnt = 0;
        for (int s = 0; s < 16; ++s) tiles[t].row[s] = -1;
    }
}

// The escapes once more, grouped by tile: entry list of tile t = the escapes of its rows in row-slot order, padded to
// an even length.  Rewrites the descriptors' e0 / e1 (absolute positions in the by-row arrays on entry) to positions
// within the tile's list.  One block.
__global__ void __launch_bounds__(1024) tile_escapes_kernel(TileDesc *__restrict__ tiles, const int *__restrict__ header,
                                                            const int *__restrict__ esc_col,
                                                            const float *__restrict__ esc_delta,
                                                            EscEntry *__restrict__ ent) {
    __shared__ int wsum[32];
    __shared__ int running;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ntiles = header[0];
    if (tid == 0) running = 0;
    __syncthreads();
    for (int t0 = 0; t0 < ntiles; t0 += 1024) {
        const int t = t0 + tid;
        int n = 0;
        if (t < ntiles)
            for (int s = 0; s < 16; ++s)
                if (tiles[t].row[s] >= 0) n += tiles[t].e1[s] - tiles[t].e0[s];
        const int np = (n + 1) & ~1;
        int incl = np;                                              // inclusive scan over the block
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += wsum[w];
        const int base = running + before + incl - np;
        if (t < ntiles) {
            TileDesc &d = tiles[t];
            d.esc0 = base;
            d.nesc = n;
            int pos = 0;
            for (int s = 0; s < 16; ++s) {
                int g0 = 0, g1 = 0;
                if (d.row[s] >= 0) { g0 = d.e0[s]; g1 = d.e1[s]; }
                d.e0[s] = pos;
                for (int e = g0; e < g1; ++e, ++pos) ent[base + pos] = EscEntry{esc_col[e], esc_delta[e]};
                d.e1[s] = pos;
            }
            if (n & 1) ent[base + n] = EscEntry{-1, 0.f};
        }
        __syncthreads();
        if (tid == 0) {
            int tot = 0;
            for (int w = 0; w < 32; ++w) tot += wsum[w];
            running += tot;
        }
        __syncthreads();
    }
}

constexpr int SMEM_JOBS = 8;   // jobs of a CTA's own range kept in shared memory
__host__ __device__ constexpr int64_t job_table_bytes(int njobs) {
    return ((int64_t)(njobs < SMEM_JOBS ? njobs : SMEM_JOBS) * 96 + 127) / 128 * 128;
}
constexpr int MAX_JOBS = 128;  // jobs behind one launch (the table travels in the kernel's parameters: 12 KB of the 32 KB
                               // a launch may carry)

struct SmallMParams {
    JobDesc jobs[MAX_JOBS];    // the launch's jobs, by value (they travel with the launch: nothing to keep alive, and a
                               // captured graph holds its own copy)
    int njobs;                 // jobs in `jobs`; with a device-resident table: its capacity
    const JobDesc *dev_jobs;   // device-resident job table (written by an earlier kernel of the stream), or null
    const int *dev_njobs;      // its length, in device memory (null: the table above is used)
    int units_per_job;         // device-resident table: every job has this many (tile, stage) units; unit0 = index x this
    float *part;               // (slots, M, Q) partial results of tiles shared by several K-ranges (single job only)
    int *ticket;               // one counter per CTA column (zero on entry, zero on exit)
    int M, MP;                 // MP: token slots per column group in shared memory (>= M)
    int S;                     // K-ranges (= gridDim.y); 1 when the launch has several jobs
    int nc_per;                // chunks per K-range (the last range may be shorter)
    int units_total;           // list launches: (tile, stage) units of all jobs
    int xs_halves;             // capacity of the staged activations in halves per layout
    int nstg;                  // slots of each pipe's copy ring
    int cps;                   // chunks per stage (a multiple of NW)
    int rs[6];                 // bytes between rows of a stage, by width 3..8
    int slot_bytes;            // a ring slot: 16 rows of the widest width
    int esc_cap;               // escape entries a side slot holds
    int debug;                 // bit 0: skip the fragment math (copy stream only); bit 1: time stamps of CTA (0, 0);
                               // bit 2: skip the row copies (math on whatever the ring holds; tuning experiments)
};

// Pipes per CTA: a pipe is four consumer warps, a producer warp and a finishing warp with a copy ring of their own.
// One CTA per SM; its pipes share the staged activations.
__host__ __device__ constexpr int pipes_for(int NT) { return NT == 1 ? PIPES_NT1 : NT == 2 ? 2 : 1; }

// Work division.  A K-range of a tile is NSK stages long.  CTA c takes a contiguous share of whole tiles (the CTAs'
// shares differ by at most one tile); the (tile, stage) units of the share, tile-major, are cut into equal runs, one
// per pipe, so that the pipes of a CTA stream the same number of bytes.  A tile cut by a run boundary is summed
// through shared memory: the pipe that holds its first stage owns it, the others contribute.
struct Visit { int tile, sb, se; };                                     // stages [sb, se) of the tile
__host__ __device__ inline void cta_tiles(int ntiles, int nctas, int c, int &t0, int &t1) {
    const int base = ntiles / nctas, extra = ntiles % nctas;
    t0 = c * base + min(c, extra);
    t1 = t0 + base + (c < extra ? 1 : 0);
}
// A pipe's run [u0, u1) as a list of visits.  Order: a run that ends inside a tile takes that (shared) tile first,
// so that the waiting a shared tile costs (fence, ticket, possibly the final sum) is hidden behind the rest of the
// run and the run ends with tiles it writes alone.
struct Run {
    int u0, u1, NSK, t_first, t_last, nv;
    bool last_first;
};
__device__ __forceinline__ Run make_run(int u0, int u1, int NSK) {
    Run r;
    r.u0 = u0; r.u1 = u1; r.NSK = NSK;
    r.nv = 0; r.t_first = r.t_last = 0; r.last_first = false;
    if (u1 > u0) {
        r.t_first = u0 / NSK;
        r.t_last = (u1 - 1) / NSK;
        r.nv = r.t_last - r.t_first + 1;
        r.last_first = r.nv > 1 && (u1 - r.t_last * NSK) < NSK;
    }
    return r;
}
__device__ __forceinline__ Visit run_visit(const Run &r, int i) {
    int j = i;                                                          // position in tile order
    if (r.last_first) j = i == 0 ? r.nv - 1 : i - 1;
    Visit v;
    v.tile = r.t_first + j;
    v.sb = j == 0 ? r.u0 - r.t_first * r.NSK : 0;
    v.se = v.tile == r.t_last ? r.u1 - r.t_last * r.NSK : r.NSK;
    return v;
}

// A warp's position in its pipe's copy ring.
struct RingPos {
    uint32_t full, empty;      // shared addresses of the current slot's barriers
    uint32_t data;             // ... and of its stage
    int slot;
    uint32_t phase;
};
__device__ __forceinline__ void ring_advance(RingPos &rp, uint32_t slot_bytes, int nstg) {
    rp.full += 8; rp.empty += 8; rp.data += slot_bytes;
    if (++rp.slot == nstg) {
        rp.full -= 8 * nstg; rp.empty -= 8 * nstg; rp.data -= slot_bytes * nstg;
        rp.slot = 0; rp.phase ^= 1u;
    }
}

// Stages [sb, se) of one tile of width NB: this warp's chunks of every stage.  CPW: chunks per warp per stage when known at compile time (0: read it from the parameters).
// Returns false if a wait gave up.
template <int NB, int NT, bool DUAL, int CPW>
__device__ __forceinline__ bool stream_tile(const SmallMParams &p, const uint32_t *pair_table, volatile int *abort_flag,
                                            RingPos &rp, int NC, int sb, int se, int warp, int lane, uint32_t xbase,
                                            uint32_t xstep, float (&acc)[NT][4]) {
    const PairConst pc = pair_const(pair_table, NB);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t RS = (uint32_t)p.rs[NB - 3];
    const uint32_t woff = (uint32_t)g * RS + (uint32_t)(t * 4 * NB) + (uint32_t)(warp * 16 * NB);
    const uint32_t xchunk = 4 * xstep;
    const int cps = CPW ? CPW * NW : p.cps;
    const int cpw = CPW ? CPW : p.cps / NW;
    const uint32_t slot_bytes = (uint32_t)p.slot_bytes;
    const int nstg = p.nstg;
    const bool math = !(p.debug & 1);
    uint32_t xptr = xbase + (uint32_t)(sb * cps + warp) * xchunk;       // this warp's first chunk of the stage
    for (int s = sb; s < se; ++s) {
        if (!mbar_wait(rp.full, rp.phase, abort_flag, 2)) return false;
        if (math) {
            const uint32_t wa = rp.data + woff;
            if ((s + 1) * cps <= NC) {                                  // a full stage
#pragma unroll
                for (int j = 0; j < (CPW ? CPW : 1); ++j) {
                    if (CPW) {
                        chunk_mma<NB, NT, DUAL>(wa + j * (NW * 16 * NB), wa + j * (NW * 16 * NB) + 8 * RS,
                                                xptr + j * NW * xchunk, xstep, acc, pc);
                    } else {
                        for (int jj = 0; jj < cpw; ++jj)
                            chunk_mma<NB, NT, DUAL>(wa + jj * (NW * 16 * NB), wa + jj * (NW * 16 * NB) + 8 * RS,
                                                    xptr + jj * NW * xchunk, xstep, acc, pc);
                    }
                }
            } else {                                                    // the K-range ends inside this stage
                for (int jj = 0; jj < cpw; ++jj)
                    if (s * cps + jj * NW + warp < NC)
                        chunk_mma<NB, NT, DUAL>(wa + jj * (NW * 16 * NB), wa + jj * (NW * 16 * NB) + 8 * RS,
                                                xptr + jj * NW * xchunk, xstep, acc, pc);
            }
        }
        xptr += (uint32_t)cps * xchunk;
        __syncwarp();
        if (lane == 0) mbar_arrive(rp.empty);
        ring_advance(rp, slot_bytes, nstg);
    }
    return true;
}

// X staging: 8 activations as saturated fp16 bit patterns, whatever the input type (runtime switch: the staging
// loop is short, and one kernel serves the three input types)
template <bool GLOBAL>
__device__ __forceinline__ void stage_x8_any(int x_dtype, const void *__restrict__ X, int64_t off, uint32_t (&h)[8], float sc) {
    if (x_dtype == QVB8_BF16) stage_x8<QVB8_BF16, GLOBAL>(X, off, h, sc);
    else if (x_dtype == QVB8_F16) stage_x8<QVB8_F16, GLOBAL>(X, off, h, sc);
    else stage_x8<QVB8_F32, GLOBAL>(X, off, h, sc);
}

// Geometry of one job for one pipe of one CTA: the CTA's share of whole tiles (CTA numbering rotated per job) and the
// pipe's run of (tile, stage) units in it.
struct JobGeom {
    int kc0, NC, NSK;          // first chunk and chunk count of this CTA's K-range; stages along K per tile
    int uc0, uc1, Lp;          // the CTA's units [uc0, uc1), units per pipe
    int ct0, ct1;              // the CTA's tiles
    Run run;                   // this pipe's run
};
struct ListShape { bool list; int units_total; };     // list = one stream of units cut into per-CTA ranges
template <int NPIPE>
__device__ __forceinline__ JobGeom job_geom(const SmallMParams &p, const ListShape &ls, const JobDesc &jd, int split, int pipe) {
    JobGeom g;
    g.kc0 = ls.list ? jd.kc0 : split * p.nc_per;
    g.NC = ls.list ? jd.nc_total : min(p.nc_per, jd.nc_total - g.kc0);
    g.NSK = (g.NC + p.cps - 1) / p.cps;
    const int nskp = jd.nsk_part > 0 ? jd.nsk_part : g.NSK;            // units per tile in the list's unit count
    if (ls.list) {
        // A list is ONE stream of (tile, stage) units, job after job, cut into equal contiguous ranges, one per CTA
        // (snapped to whole tiles: a tile goes to the CTA that holds its first unit).  A CTA therefore meets only the
        // one or two jobs its range touches, stages activations that often, and all CTAs finish together.
        const int64_t lo = (int64_t)blockIdx.x * ls.units_total / gridDim.x - jd.unit0;
        const int64_t hi = (int64_t)(blockIdx.x + 1) * ls.units_total / gridDim.x - jd.unit0;
        const int64_t t0 = lo <= 0 ? 0 : (lo + nskp - 1) / nskp, t1 = hi <= 0 ? 0 : (hi + nskp - 1) / nskp;
        g.ct0 = (int)(t0 < jd.ntiles ? t0 : jd.ntiles);
        g.ct1 = (int)(t1 < jd.ntiles ? t1 : jd.ntiles);
    } else {
        cta_tiles(jd.ntiles, gridDim.x, blockIdx.x, g.ct0, g.ct1);
    }
    g.uc0 = g.ct0 * g.NSK;
    g.uc1 = g.ct1 * g.NSK;
    g.Lp = max(1, (g.uc1 - g.uc0 + NPIPE - 1) / NPIPE);
    const int u0 = min(g.uc0 + pipe * g.Lp, g.uc1), u1 = min(u0 + g.Lp, g.uc1);
    g.run = make_run(u0, u1, g.NSK);
    return g;
}

// Stages this consumer warp's slice of a job's activations (all tokens) as saturated fp16 in MMA fragment order (layout
// A, and layout B when DUAL) and leaves the slice's per-token sums in psum_w[m].  X points at row 0 of the (M, P)
// activations: global memory (GLOBAL) or the raw copy in shared memory.  Warp cw of ncw takes the 8-column groups
// [cw * per, (cw + 1) * per) of the K-range.  Sums run over the narrowed values in a fixed order (same bits every run).
template <bool DUAL, bool GLOBAL, typename ScaleOf>
__device__ __forceinline__ void stage_slice(const void *X, int x_dtype, int64_t ldx, int kc0, int NC, int M, int MP,
                                            __half *xs_a, __half *xs_b, int cw, int ncw, int lane, ScaleOf sc_of,
                                            float *psum_w) {
    const int groups = NC * 16;
    const int per = (groups + ncw - 1) / ncw;
    const int g0 = cw * per, g1 = min(groups, g0 + per);
    const int64_t col0 = (int64_t)kc0 * KC;
    constexpr int UNR = 4;                                              // loads in flight per thread
    if (per <= 32 && MP > 1) {
        // At most one column group per lane: the loads of four TOKENS are in flight together (with the loop below every
        // token would be one round trip to memory).  The same arithmetic per token, hence the same bits.
        const int u8 = g0 + lane;
        const bool on = u8 < g1;
        for (int m0 = 0; m0 < MP; m0 += UNR) {
            uint32_t h[UNR][8];
#pragma unroll
            for (int i = 0; i < UNR; ++i) {
                const int m = m0 + i;
                if (on && m < M) {
                    stage_x8_any<GLOBAL>(x_dtype, X, (int64_t)m * ldx + col0 + (int64_t)u8 * 8, h[i], sc_of(m));
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) h[i][j] = 0u;
                }
            }
#pragma unroll
            for (int i = 0; i < UNR; ++i) {
                const int m = m0 + i;
                if (m >= MP) break;
                float s = 0.f;
                if (on) {
                    const int sl = slot_of(u8 * 8, m, MP);
                    *reinterpret_cast<uint4 *>(xs_a + (sl << 3)) = make_uint4(
                        h[i][0] | (h[i][2] << 16), h[i][1] | (h[i][3] << 16), h[i][4] | (h[i][6] << 16), h[i][5] | (h[i][7] << 16));
                    if (DUAL)
                        *reinterpret_cast<uint4 *>(xs_b + (sl << 3)) = make_uint4(
                            h[i][0] | (h[i][4] << 16), h[i][1] | (h[i][5] << 16), h[i][2] | (h[i][6] << 16), h[i][3] | (h[i][7] << 16));
#pragma unroll
                    for (int j = 0; j < 8; ++j) s += __half2float(__ushort_as_half((unsigned short)h[i][j]));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0 && m < M) psum_w[m] = s;
            }
        }
        return;
    }
    for (int m = 0; m < MP; ++m) {
        float s = 0.f;
        const float sc = m < M ? sc_of(m) : 1.f;
        for (int base = g0 + lane; base < g1; base += 32 * UNR) {
            uint32_t h[UNR][8];
#pragma unroll
            for (int i = 0; i < UNR; ++i) {
                const int u8 = base + i * 32;
                if (u8 < g1 && m < M) {
                    stage_x8_any<GLOBAL>(x_dtype, X, (int64_t)m * ldx + col0 + (int64_t)u8 * 8, h[i], sc);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) h[i][j] = 0u;
                }
            }
#pragma unroll
            for (int i = 0; i < UNR; ++i) {
                const int u8 = base + i * 32;
                if (u8 >= g1) continue;
                const int sl = slot_of(u8 * 8, m, MP);
                *reinterpret_cast<uint4 *>(xs_a + (sl << 3)) = make_uint4(
                    h[i][0] | (h[i][2] << 16), h[i][1] | (h[i][3] << 16), h[i][4] | (h[i][6] << 16), h[i][5] | (h[i][7] << 16));
                if (DUAL)
                    *reinterpret_cast<uint4 *>(xs_b + (sl << 3)) = make_uint4(
                        h[i][0] | (h[i][4] << 16), h[i][1] | (h[i][5] << 16), h[i][2] | (h[i][6] << 16), h[i][3] | (h[i][7] << 16));
#pragma unroll
                for (int j = 0; j < 8; ++j) s += __half2float(__ushort_as_half((unsigned short)h[i][j]));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0 && m < M) psum_w[m] = s;
    }
}

// Completion number n of a barrier that completes once per use -> the parity a waiter passes.
__device__ __forceinline__ uint32_t par(int n) { return (uint32_t)(n & 1); }

// DUAL: a second activation layout is staged for widths that pair ids at distance 4 (cheap for few tokens).
// NPIPE: pipes per CTA.  Four stream fastest; a two-pipe CTA is small enough (threads, registers, shared memory) for
// the next kernel's CTA to sit beside it and run its prologue early (a tuning switch, see make_plan).
//
// A launch runs a LIST of jobs (products) back to back inside the CTAs: the copy rings, barriers and warp roles
// persist from one job to the next, so the stream of weight bytes never drains between jobs.  A list is cut into one
// contiguous range of tiles per CTA, so a CTA crosses a job boundary once or twice per launch; there all its consumer
// warps meet and stage the next job's activations.  The jobs must not depend
// on one another's outputs.  A launch with one job is the plain product.
template <int NT, bool DUAL, int NPIPE>
__global__ void __launch_bounds__(NPIPE * PIPE_THREADS, 1) small_m_kernel(const __grid_constant__ SmallMParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ Control ctl;
    constexpr int RED_FLOATS = NW * 4 * NT * 32;                       // a pipe's hand-over buffer (>= 16 * M floats)
    constexpr int CWARPS = NPIPE * NW;                                 // consumer warps of the CTA

    const int tid = threadIdx.x, lane = tid & 31;
    const int pipe = tid / PIPE_THREADS, warp = (tid % PIPE_THREADS) >> 5;     // warp: role within the pipe
    const int split = blockIdx.y;
    const int cps = p.cps;
    const int MP = p.MP, M = p.M;
    const int nstg = p.nstg;
    // A device-resident job table was written by the kernel before this one in the stream: wait for it first.
    const bool devlist = p.dev_njobs != nullptr;
    if (devlist) pdl_wait();
    const int njobs = devlist ? min(__ldg(p.dev_njobs), p.njobs) : p.njobs;
    if (njobs <= 0) return;                                            // (an empty device-resident table: nothing to do)
    const JobDesc *jtab = devlist ? p.dev_jobs : p.jobs;
    const ListShape ls{devlist || njobs > 1, devlist ? njobs * p.units_per_job : p.units_total};
    // dynamic shared memory:
    //   [job table] [activations: layout A, layout B] [16 zero bytes, padded to 128]
    //   [activation sums by consumer warp, two sets] [exchange buffers of tiles shared by pipes]
    //   per pipe: [ring: nstg stages of 16 rows] [side ring: NSIDE x (descriptor + escapes)] [two hand-over buffers]
    //             [escape corrections]
    // The table in shared memory holds only the jobs THIS CTA's range touches (a list's CTA meets one or two; SMEM_JOBS
    // at most -- a range that touches more reads the launch's table where it lies).
    JobDesc *jobs_sm = reinterpret_cast<JobDesc *>(smem);
    const size_t jobs_bytes = (size_t)job_table_bytes(p.njobs);
    __half *xs_a = reinterpret_cast<__half *>(smem + jobs_bytes);
    __half *xs_b = DUAL ? xs_a + p.xs_halves : xs_a;
    uint32_t *zero16 = reinterpret_cast<uint32_t *>(xs_a + (DUAL ? 2 : 1) * p.xs_halves);
    float *psum = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(zero16) + 128);   // [2][CWARPS][M]
    const size_t psum_bytes = (size_t)((2 * CWARPS * M * 4 + 127) / 128 * 128);
    const int xch_floats = 16 * M;                                     // one tile's results
    float *xch = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(psum) + psum_bytes);   // [owner][contributor][16][M]
    float *own = xch + XCH_SLOTS * xch_floats;                                 // [NPIPE][16][M]: an owner's own part of its shared tile
    const size_t shared_bytes = (size_t)(((XCH_SLOTS + NPIPE) * xch_floats * 4 + 127) / 128 * 128);
    const int esc_cap = p.esc_cap;
    const int side_bytes = (int)side_slot_bytes(esc_cap);
    const size_t pipe_bytes = (size_t)nstg * p.slot_bytes + (size_t)NSIDE * side_bytes + (size_t)2 * RED_FLOATS * 4 +
                              (size_t)corr_bytes(M, esc_cap);
    uint8_t *pbase = reinterpret_cast<uint8_t *>(xch) + shared_bytes + (size_t)pipe * pipe_bytes;
    uint8_t *side = pbase + (size_t)nstg * p.slot_bytes;               // [NSIDE][side_bytes]
    float *red = reinterpret_cast<float *>(side + NSIDE * side_bytes); // [2][NW][4 * NT][32]
    float *corr = red + 2 * RED_FLOATS;                                // [16][M], private to the finishing warp
    PipeControl &pc_ = ctl.pipe[pipe];
    volatile int *abort_flag = &ctl.abort;
    const bool tracer = (p.debug & 2) && pipe == 0;

    if (tracer) trace(p.debug, 0);
    // the jobs this CTA's range touches: jfirst .. jend - 1 (a list's ranges are contiguous); every warp walks the same
    // sequence and counts its barrier phases by the position in it.  Read from the launch parameters: the shared-memory
    // copy of the job table is not there yet, and the producer wants its first descriptor on the way before anything else.
    int jfirst = 0, jcount = njobs;
    if (ls.list) {
        const int64_t lo = (int64_t)blockIdx.x * ls.units_total / gridDim.x, hi = (int64_t)(blockIdx.x + 1) * ls.units_total / gridDim.x;
        int j = 0;
        if (devlist) {
            j = min(njobs - 1, (int)(lo / max(1, p.units_per_job)));
        } else {
            // the job that holds the range's first unit (the first K-range of its pack): unit0 never decreases along
            // the table, so a bisection finds the last job with unit0 <= lo, and a short walk back its pack's first range
            int a = 0, b = njobs - 1;
            while (a < b) {
                const int mid = (a + b + 1) >> 1;
                if (jtab[mid].unit0 <= lo) a = mid; else b = mid - 1;
            }
            while (a > 0 && jtab[a - 1].unit0 == jtab[a].unit0) --a;
            j = a;
        }
        int jlast = -1;
        jfirst = njobs;
        for (; j < njobs && jtab[j].unit0 < hi; ++j) {
            const JobGeom gj = job_geom<NPIPE>(p, ls, jtab[j], split, 0);
            if (gj.ct1 > gj.ct0) { if (j < jfirst) jfirst = j; jlast = j; }
        }
        jcount = jlast >= jfirst ? jlast - jfirst + 1 : 0;
        if (jcount == 0) jfirst = 0;
    }
    const int jend = jfirst + jcount;
    // the producer's first descriptor fields are on their way from memory while the barriers are set up
    int pf_nb = 0, pf_cnt = 0, pf_esc0 = 0, pf_nesc = 0, pf_j = -1, pf_i = 0;
    uint32_t pf_b16 = 0;
    if (warp == PRODUCER_WARP) {
        for (int j = jfirst; j < jend && pf_j < 0; ++j) {
            const JobGeom gj = job_geom<NPIPE>(p, ls, jtab[j], split, pipe);
            if (gj.run.nv > 0) {
                const TileDesc *d = jtab[j].tiles + run_visit(gj.run, 0).tile;
                pf_nb = __ldg(&d->nb);
                pf_cnt = __ldg(&d->cnt);
                pf_esc0 = __ldg(&d->esc0);
                pf_nesc = __ldg(&d->nesc);
                pf_b16 = lane < 16 ? __ldg(&d->b16[lane]) : 0u;
                pf_j = j;
            }
        }
    }
    // the CTA's jobs: from the launch parameters (or the device-resident table) into shared memory, where every warp
    // reads them at each job boundary; indexed by job number like the table they come from
    const bool table_in_smem = jcount <= SMEM_JOBS;
    const JobDesc *jobs = table_in_smem ? jobs_sm - jfirst : jtab;
    if (table_in_smem) {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(jtab + jfirst);
        uint32_t *dst = reinterpret_cast<uint32_t *>(jobs_sm);
        for (int i = tid; i < jcount * (int)(sizeof(JobDesc) / 4); i += blockDim.x) dst[i] = src[i];
    }
    // barriers: one thread each
    {
        const int per_pipe = 2 * nstg + 2 * NSIDE + 4;
        if (tid < NPIPE * per_pipe) {
            PipeControl &q = ctl.pipe[tid / per_pipe];
            const int k = tid % per_pipe;
            if (k < nstg) mbar_init(smem_u32(&q.full[k]), 1);
            else if (k < 2 * nstg) mbar_init(smem_u32(&q.empty[k - nstg]), NW);
            else if (k < 2 * nstg + NSIDE) mbar_init(smem_u32(&q.side_full[k - 2 * nstg]), 1);
            else if (k < 2 * nstg + 2 * NSIDE) mbar_init(smem_u32(&q.side_empty[k - 2 * nstg - NSIDE]), NW + 1);
            else if (k < 2 * nstg + 2 * NSIDE + 2) mbar_init(smem_u32(&q.red_full[k - 2 * nstg - 2 * NSIDE]), NW);
            else mbar_init(smem_u32(&q.red_empty[k - 2 * nstg - 2 * NSIDE - 2]), 1);
        } else if (tid < NPIPE * per_pipe + XCH_SLOTS) {
            mbar_init(smem_u32(&ctl.xch_full[tid - NPIPE * per_pipe]), 1);
            mbar_init(smem_u32(&ctl.xch_empty[tid - NPIPE * per_pipe]), 1);
        } else if (tid == NPIPE * per_pipe + XCH_SLOTS) {
            mbar_init(smem_u32(&ctl.amax_ready), CWARPS);
            mbar_init(smem_u32(&ctl.x_ready), CWARPS);
            mbar_init(smem_u32(&ctl.job_done), CWARPS);
            mbar_init(smem_u32(&ctl.fin_started), NPIPE);
            ctl.abort = 0;
        }
        if (tid <= NPIPE * per_pipe + XCH_SLOTS) asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (tid >= 152 && tid < 156) zero16[tid - 152] = 0u;
    if (tid >= 128 && tid < 128 + PAIR_TABLE_WORDS) ctl.pair_table[tid - 128] = pair_const_word(3 + ((tid - 128) >> 2), (tid - 128) & 3);
    if (tid < MAX_M) { ctl.amax[tid] = 0u; ctl.kexp[tid] = 0; }                       // (the smallest CTA has 192 threads)
    __syncthreads();
    pdl_launch_dependents();                                            // what follows in the stream may start its own prologue
    if (tracer) trace(p.debug, 1);
    RingPos rp;
    rp.full = smem_u32(&pc_.full[0]); rp.empty = smem_u32(&pc_.empty[0]); rp.data = smem_u32(pbase);
    rp.slot = 0; rp.phase = 0;
    const uint32_t side_full0 = smem_u32(&pc_.side_full[0]), side_empty0 = smem_u32(&pc_.side_empty[0]);

    if (warp == PRODUCER_WARP) {
        // ================= producer warp: per visit, lane 16 copies the tile's descriptor and lane 17 its escapes into
        // a side slot; per stage, lane r copies row r.  The next visit's descriptor fields are fetched one visit
        // ahead, across job boundaries too =================
        bool alive = true;
        int nb = 0, cnt = 0, esc0 = 0, nesc = 0;
        uint32_t b16 = 0;
        // cursor over (job, visit) pairs that exist
        int cj = jfirst, ci = -1;
        JobGeom cg = job_geom<NPIPE>(p, ls, jobs[jfirst], split, pipe);
        if (jcount == 0) cg.run.nv = 0;
        auto advance = [&](int &j, int &i, JobGeom &g) {                // -> false when the list is exhausted
            ++i;
            while (i >= g.run.nv) {
                if (++j >= jend) return false;
                g = job_geom<NPIPE>(p, ls, jobs[j], split, pipe);
                i = 0;
            }
            return true;
        };
        auto fetch = [&](int j, int i, const JobGeom &g) {
            const TileDesc *d = jobs[j].tiles + run_visit(g.run, i).tile;
            nb = __ldg(&d->nb);
            cnt = __ldg(&d->cnt);
            esc0 = __ldg(&d->esc0);
            nesc = __ldg(&d->nesc);
            b16 = lane < 16 ? __ldg(&d->b16[lane]) : 0u;
        };
        bool have = advance(cj, ci, cg);
        if (have) {
            if (cj == pf_j && ci == pf_i) { nb = pf_nb; cnt = pf_cnt; esc0 = pf_esc0; nesc = pf_nesc; b16 = pf_b16; }
            else fetch(cj, ci, cg);
        }
        if (tracer) trace(p.debug, 2);
        const bool nocopy = (p.debug & 4) != 0;
        const uint64_t stream_policy = l2_evict_first_policy();
        int vis = 0;                                                    // visits issued so far (all jobs)
        while (have && alive) {
            const JobDesc &jd = jobs[cj];
            const Visit v = run_visit(cg.run, ci);
            const int NC = cg.NC, kc0 = cg.kc0;
            const int cnb = nb, ccnt = cnt;
            const bool planned = jd.esc_ent != nullptr && !(jd.yflags & 1);   // (a pre-pass has applied the job's escapes)
            const uint32_t ebytes = planned ? (uint32_t)(min((nesc + 1) & ~1, esc_cap) * 8) : 0u;   // (in-line: yflags bit 2)
            const EscEntry *esrc = jd.esc_ent + esc0;
            const uint32_t step = (uint32_t)(cps * 16 * cnb);           // bytes of a row per full stage
            const uint8_t *src = jd.ids + ((uint64_t)b16 + (uint64_t)kc0 * cnb) * 16u + (size_t)v.sb * step;
            const TileDesc *dsrc = jd.tiles + v.tile;
            // next visit's descriptor loads while this visit is issued
            int nj = cj, ni = ci;
            JobGeom ng = cg;
            const bool more = advance(nj, ni, ng);
            if (more) fetch(nj, ni, ng);
            // descriptor and escapes
            const int sslot = vis % NSIDE;
            if (!mbar_wait(side_empty0 + 8 * sslot, par(vis / NSIDE) ^ 1u, abort_flag, 7, 200)) { alive = false; break; }
            const uint32_t sfull = side_full0 + 8 * sslot, sdst = smem_u32(side + sslot * side_bytes);
            if (lane == 0) mbar_expect_tx(sfull, (uint32_t)DESC_BYTES + ebytes);
            __syncwarp();
            if (lane == 16) bulk_g2s(sdst, dsrc, DESC_BYTES, sfull);
            if (lane == 17 && ebytes) bulk_g2s(sdst + DESC_SLOT, esrc, ebytes, sfull);
            // rows (a per-element tile has none: its rows are read from global memory)
            const uint32_t dst_row = (uint32_t)(lane * (cnb ? p.rs[cnb - 3] : 0));
            const int s_end = cnb ? v.se : v.sb;
            for (int s = v.sb; s < s_end; ++s) {
                const int chunks = min(cps, NC - s * cps);
                const uint32_t bytes_row = nocopy ? 0u : (uint32_t)(chunks * 16 * cnb);
                if (!mbar_wait(rp.empty, rp.phase ^ 1u, abort_flag, 1, 100)) { alive = false; break; }
                if (lane == 0) mbar_expect_tx(rp.full, bytes_row * (uint32_t)ccnt);
                __syncwarp();
                if (bytes_row && lane < ccnt) {
                    if (p.debug & 16) bulk_g2s(rp.data + dst_row, src, bytes_row, rp.full);
                    else bulk_g2s_stream(rp.data + dst_row, src, bytes_row, rp.full, stream_policy);
                }
                src += step;
                if (tracer && vis == 0 && s == v.sb) trace(p.debug, 3);
                ring_advance(rp, (uint32_t)p.slot_bytes, nstg);
            }
            ++vis;
            cj = nj; ci = ni; cg = ng; have = more;
        }
        // nothing may be in flight when the CTA exits: wait until every issued stage and side slot has been consumed
        for (int s = 0; s < nstg && alive; ++s) {
            alive = mbar_wait(rp.empty, rp.phase ^ 1u, abort_flag, 1, 200);
            ring_advance(rp, (uint32_t)p.slot_bytes, nstg);
        }
        for (int k = 0; k < NSIDE && alive; ++k) {
            const int i = vis + k;                                      // as if about to reuse the slot
            alive = mbar_wait(side_empty0 + 8 * (i % NSIDE), par(i / NSIDE) ^ 1u, abort_flag, 7);
        }
        if (!alive) {
            // a wait gave up somewhere: copies may still be in flight towards this CTA's shared memory; keep the CTA
            // resident until any such copy (a few kilobytes at most) has certainly landed
            const uint64_t t0 = global_ns();
            while (global_ns() - t0 < 200000ull) {}
        }
    } else if (warp == FINISHER_WARP) {
        // ================= finishing warp: per visit, sums the escape corrections of its rows while the stages stream,
        // then takes the consumer warps' partial sums, scales, corrects and writes the rows =================
        const int g = lane >> 2, t = lane & 3;
        bool alive = true;
        int vis = 0;                                                    // visits handled so far (all jobs)
        int own_uses[MAX_PIPES - 1] = {0, 0, 0};                        // completions waited for on this pipe's xch_full[j]
        int give_uses[MAX_PIPES - 1] = {0, 0, 0};                       // parts handed to owner pipe op (index op)
        for (int kj = 0; kj < jcount; ++kj) {
            const int job = jfirst + kj;
            const JobDesc &jd = jobs[job];
            const JobGeom gm = job_geom<NPIPE>(p, ls, jd, split, pipe);
            const Run &run = gm.run;
            const int kc0 = gm.kc0, NC = gm.NC, NSK = gm.NSK;
            const __half *xsa = xs_a;
            const bool inline_esc = jd.esc_ent != nullptr && (jd.yflags & 4);   // a consumer warp sums each tile's corrections
            const bool planned = jd.esc_ent != nullptr && !(jd.yflags & 5);   // escapes corrected here (else: pre-pass / in-line)
            const bool add_to_y = jd.esc_ent != nullptr && (jd.yflags & 1);   // Y holds the pre-pass's corrections: add to it
            const bool later_range = (jd.yflags & 2) != 0;                 // Y holds this thread's sums of the earlier K-ranges
            const bool prescaled = njobs == 1 && jd.x_mode == 1 && jd.x_dtype != QVB8_F16;
            // the job's activations are staged and every consumer warp has left its partial sums of them: this lane
            // keeps the sums of the tokens it writes (8n + 2t + k), added up in warp order (same bits every run)
            if (alive) alive = mbar_wait(smem_u32(&ctl.x_ready), par(kj), abort_flag, 5);
            float sumx_nt[NT][2];
            {
                const float *ps = psum + (kj & 1) * CWARPS * M;
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int m = 8 * n + 2 * t + k;
                        float sx = 0.f;
                        if (m < M)
                            for (int w = 0; w < CWARPS; ++w) sx += ps[w * M + m];
                        sumx_nt[n][k] = sx;
                    }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl.fin_started));
            int own_contrib = 0, own_row[2] = {-1, -1};
            // writes a finished tile (of this K-range): the result itself, or with several K-ranges a partial result; the
            // K-ranges' partial results of all of a CTA's tiles are added up in range order at the end of the kernel
            auto emit_tile = [&](const int (&rows)[2], const float (&y)[2][NT][2]) {
                float *out = p.S == 1 ? jd.Y : p.part + (int64_t)split * M * jd.Q;
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int m = 8 * n + 2 * t + k;
                            if (rows[hrow] >= 0 && m < M) {
                                float *dst = out + (int64_t)m * jd.Q + rows[hrow];
                                // after a pre-pass: one atomic addition per element and K-range; the ranges of a pack are
                                // added by the same thread in program order, so the sum has one order
                                if (add_to_y) atomicAdd(dst, y[hrow][n][k]);
                                else if (later_range) *dst += y[hrow][n][k];
                                else *dst = y[hrow][n][k];
                            }
                        }
            };
            for (int i = 0; i < run.nv; ++i, ++vis) {
                const Visit v = run_visit(run, i);
                // ---- the tile's descriptor and escapes arrive in a side slot
                const int sslot = vis % NSIDE;
                const bool fstamp = tracer && (p.debug & 64) && vis >= 4 && vis < 8;   // tuning: time stamps of visits 4..7
                if (fstamp) trace(p.debug, 16 + 4 * (vis - 4));
                if (alive) alive = mbar_wait(side_full0 + 8 * sslot, par(vis / NSIDE), abort_flag, 8, 200);
                if (fstamp) trace(p.debug, 17 + 4 * (vis - 4));
                const TileDesc *d = reinterpret_cast<const TileDesc *>(side + sslot * side_bytes);
                const EscEntry *ent = reinterpret_cast<const EscEntry *>(side + sslot * side_bytes + DESC_SLOT);
                int cnb = 0, myrow[2] = {-1, -1};
                float myms[2] = {0.f, 0.f}, myts[2] = {0.f, 0.f};
                if (alive) {
                    cnb = d->nb;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        myrow[h] = d->row[g + 8 * h];
                        myms[h] = d->ms[g + 8 * h];
                        myts[h] = d->ts[g + 8 * h];
                    }
                }
                // ---- escapes: lane r sums row r's corrections x * (exact - band), in stored order, over the visit's columns
                if (planned && alive && M == 1) {
                    // One token: the per-entry work (column test, activation fetch) is spread over all 32 lanes first; the
                    // row's sum then runs over (difference, activation) pairs in stored order with the same fused
                    // multiply-adds as below, so the result has the same bits.  This warp shares its scheduler with
                    // issue-bound consumer warps: a long serial loop here ends after the stream and delays the CTA's end.
                    const int clo = (kc0 + v.sb * cps) * KC, chi = (kc0 + min(v.se * cps, NC)) * KC, cbase = kc0 * KC;
                    float2 *pd = reinterpret_cast<float2 *>(reinterpret_cast<uint8_t *>(corr) + corr_buffers(M) * corr_stride_bytes(M));
                    const int ne = min(d->nesc, esc_cap);
                    for (int e = lane; e < ne; e += 32) {
                        const EscEntry en = ent[e];
                        float2 r = make_float2(0.f, 0.f);
                        if (en.col >= clo && en.col < chi) {
                            const int cc = en.col - cbase;
                            r = make_float2(en.delta, __half2float(xsa[((size_t)slot_of(cc, 0, MP) << 3) + pos_a(cc & 7)]));
                        }
                        pd[e] = r;
                    }
                    __syncwarp();
                    if (lane < 16 && d->row[lane] >= 0) {
                        const int ce0 = d->e0[lane], ce1 = d->e1[lane];
                        const EscEntry *gent = jd.esc_ent + d->esc0;
                        float a = 0.f;
                        for (int e = ce0; e < ce1; ++e) {
                            if (e < esc_cap) {
                                const float2 r = pd[e];
                                a = __fmaf_rn(r.y, r.x, a);
                            } else {
                                const int col = __ldg(&gent[e].col);
                                if (col >= clo && col < chi) {
                                    const int cc = col - cbase;
                                    a = __fmaf_rn(__half2float(xsa[((size_t)slot_of(cc, 0, MP) << 3) + pos_a(cc & 7)]), __ldg(&gent[e].delta), a);
                                }
                            }
                        }
                        corr[lane * M] = a;
                    }
                } else if (planned && alive) {
                    const int clo = (kc0 + v.sb * cps) * KC, chi = (kc0 + min(v.se * cps, NC)) * KC, cbase = kc0 * KC;
                    if (lane < 16 && d->row[lane] >= 0) {
                        const int ce0 = d->e0[lane], ce1 = d->e1[lane];
                        const EscEntry *gent = jd.esc_ent + d->esc0;    // the same list in global memory (for the overflow)
                        float *dst = corr + lane * M;
                        for (int m0 = 0; m0 < M; m0 += 8) {
                            float a[8];
#pragma unroll
                            for (int k = 0; k < 8; ++k) a[k] = 0.f;
                            for (int e = ce0; e < ce1; ++e) {
                                EscEntry en;
                                if (e < esc_cap) en = ent[e];
                                else { en.col = __ldg(&gent[e].col); en.delta = __ldg(&gent[e].delta); }
                                if (en.col >= clo && en.col < chi) {
                                    // the column's activations of consecutive tokens lie four slots (32 halves) apart
                                    const int cc = en.col - cbase;
                                    const __half *xp = xsa + ((size_t)slot_of(cc, m0, MP) << 3) + pos_a(cc & 7);
#pragma unroll
                                    for (int k = 0; k < 8; ++k)
                                        if (m0 + k < M) a[k] = __fmaf_rn(__half2float(xp[k * 32]), en.delta, a[k]);
                                }
                            }
#pragma unroll
                            for (int k = 0; k < 8; ++k)
                                if (m0 + k < M) dst[m0 + k] = a[k];
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(side_empty0 + 8 * sslot);    // done with the side slot
                if (tracer && vis == 0) trace(p.debug, 9);
                // ---- the consumer warps' partial sums (or, for a per-element tile, complete row results): taken into
                // registers and the buffer handed straight back
                const int rb = vis & 1;
                const float *redb = red + rb * RED_FLOATS;
                if (alive) alive = mbar_wait(smem_u32(&pc_.red_full[rb]), par(vis / 2), abort_flag, 3, 200);
                if (tracer && vis == 0) trace(p.debug, 10);
                if (fstamp) trace(p.debug, 18 + 4 * (vis - 4));
                float acc[NT][4];
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float a = 0.f;
                        if (cnb != 0) {
#pragma unroll
                            for (int w = 0; w < NW; ++w) a += redb[(w * 4 * NT + n * 4 + k) * 32 + lane];
                        } else {
                            // k = 2 * hrow + kk  ->  row g + 8 * hrow, token 8n + 2t + kk
                            const int m = 8 * n + 2 * t + (k & 1);
                            if (m < M) a = redb[(g + 8 * (k >> 1)) * M + m];
                        }
                        acc[n][k] = a;
                    }
                // in-line escapes: the visit's corrections lie in the correction buffers of the same parity, one partial
                // sum per consumer warp, written before the warps handed over their sums
                float cin[NT][4];
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int m = 8 * n + 2 * t + (k & 1);
                        float c = 0.f;
                        if (inline_esc && m < M) {
                            const float *cw = corr + rb * NW * (int)(corr_stride_bytes(M) / 4) + (g + 8 * (k >> 1)) * M + m;
#pragma unroll
                            for (int w = 0; w < NW; ++w) c += cw[w * (int)(corr_stride_bytes(M) / 4)];   // warp order
                        }
                        cin[n][k] = c;
                    }
                __syncwarp();                                           // every lane is done with the buffers
                if (lane == 0) mbar_arrive(smem_u32(&pc_.red_empty[rb]));
                // y = tau_s * sum(x * id) + min_s * sum(x) + corrections for rows g, g+8 and tokens 8n+2t, 8n+2t+1
                // (per-element rows arrive complete); the min_s term goes with the visit that holds the first stage
                float y[2][NT][2];
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int m = 8 * n + 2 * t + k;
                            float val = acc[n][2 * hrow + k];
                            if (myrow[hrow] >= 0 && m < M) {
                                if (cnb != 0) {
                                    val *= myts[hrow];
                                    if (v.sb == 0) val = __fmaf_rn(myms[hrow], sumx_nt[n][k], val);
                                }
                                if (planned) val += corr[(g + 8 * hrow) * M + m];
                                if (inline_esc) val += cin[n][2 * hrow + k];
                                if (prescaled) val *= pow2f(ctl.kexp[m]);
                            }
                            y[hrow][n][k] = val;
                        }
                __syncwarp();                                           // every lane is done with corr
                // a tile cut by run boundaries: the pipe that holds its first stage owns it, the later pipes hand their
                // parts over in shared memory; the owner adds them up when its run is done
                const bool partial = !(v.sb == 0 && v.se == NSK);
                bool emit = true;
                if (partial) {
                    const int op = (v.tile * NSK - gm.uc0) / gm.Lp;     // the pipe that holds the tile's first stage
                    float *dst;
                    if (op == pipe) {
                        dst = own + pipe * xch_floats;
                        own_contrib = min((v.tile * NSK + NSK - 1 - gm.uc0) / gm.Lp, NPIPE - 1) - op;
                        own_row[0] = myrow[0]; own_row[1] = myrow[1];
                    } else {
                        // the exchange slot is reused from job to job: the owner must have taken the previous part
                        const int xs = op * (MAX_PIPES - 1) + (pipe - op - 1);
                        if (give_uses[op] > 0 && alive)
                            alive = mbar_wait(smem_u32(&ctl.xch_empty[xs]), par(give_uses[op] - 1), abort_flag, 9, 100);
                        ++give_uses[op];
                        dst = xch + xs * xch_floats;
                    }
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow)
#pragma unroll
                        for (int n = 0; n < NT; ++n)
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const int m = 8 * n + 2 * t + k;
                                if (m < M) dst[(g + 8 * hrow) * M + m] = y[hrow][n][k];
                            }
                    if (op != pipe) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&ctl.xch_full[op * (MAX_PIPES - 1) + (pipe - op - 1)]));
                    }
                    emit = false;
                }
                if (tracer && vis == 0) trace(p.debug, 11);
                if (emit) emit_tile(myrow, y);
                if (tracer && vis == 0) trace(p.debug, 12);
                if (fstamp) trace(p.debug, 19 + 4 * (vis - 4));
            }
            // ---- the tile this pipe shares with later pipes: their parts have long arrived
            if (own_contrib > 0) {
                for (int j = 0; j < own_contrib; ++j) {
                    if (alive) alive = mbar_wait(smem_u32(&ctl.xch_full[pipe * (MAX_PIPES - 1) + j]), par(own_uses[j]), abort_flag, 9);
                    ++own_uses[j];
                }
                float y[2][NT][2];
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int m = 8 * n + 2 * t + k;
                            float val = 0.f;
                            if (m < M) {
                                const int o = (g + 8 * hrow) * M + m;
                                val = own[pipe * xch_floats + o];
                                for (int j = 0; j < own_contrib; ++j) val += xch[(pipe * (MAX_PIPES - 1) + j) * xch_floats + o];
                            }
                            y[hrow][n][k] = val;
                        }
                __syncwarp();                                           // every lane has read the parts
                if (lane == 0)
                    for (int j = 0; j < own_contrib; ++j) mbar_arrive(smem_u32(&ctl.xch_empty[pipe * (MAX_PIPES - 1) + j]));
                if (alive) emit_tile(own_row, y);
            }
        }
        if (tracer) trace(p.debug, 13);
    } else {
        // ================= consumer warps =================
        const int g = lane >> 2, t = lane & 3;
        const bool xvalid = NT > 1 || g < MP;                           // lanes whose token slot exists
        const uint32_t xstep = xvalid ? (uint32_t)(4 * MP * 16) : 0u;   // bytes between consecutive 8-column groups
        const uint32_t xoff = (uint32_t)((g * 4 + t) * 16);
        const int cpw = cps / NW;
        bool alive = true;
        int vis = 0;                                                    // visits walked so far (all jobs)
        const int cwarp = pipe * NW + warp;                             // index among the CTA's consumer warps
        for (int kj = 0; kj < jcount && alive; ++kj) {
            const int job = jfirst + kj;
            const JobDesc &jd = jobs[job];
            const JobGeom gm = job_geom<NPIPE>(p, ls, jd, split, pipe);
            const Run &run = gm.run;
            const int kc0 = gm.kc0, NC = gm.NC;
            const bool inline_esc = jd.esc_ent != nullptr && (jd.yflags & 4);   // this job's escapes are summed here
            float *psum_w = psum + ((kj & 1) * CWARPS + cwarp) * M;
            if (kj == 0) {
                // ---- activations of the first job's K-range as fp16 in fragment order (after the previous kernel in the
                // stream): all consumer warps of the CTA share the work, every one of them reads all of it afterwards
                pdl_wait();
                if (tracer && warp == 0) trace(p.debug, 4);
                const int ctid = cwarp * 32 + lane;                     // index among the consumer threads
                constexpr int CTHREADS = CWARPS * 32;
                // x_mode 1 (activations beyond the fp16 range): a first pass finds every token's largest magnitude in this
                // K-range; the token is then staged times 2^-k, k the smallest exponent that brings it into range, and its
                // results are multiplied by 2^k on the way out -- both exact.  fp16 input needs no prescale.
                const bool prescale = njobs == 1 && jd.x_mode == 1 && jd.x_dtype != QVB8_F16;
                if (prescale) {
                    const int groups = NC * 16, total = MP * groups;
                    const int64_t col0 = (int64_t)kc0 * KC;
                    for (int idx = ctid; idx < total; idx += CTHREADS) {
                        const int m = idx / groups, u8 = idx - m * groups;
                        if (m < M) {
                            const int64_t off = (int64_t)m * jd.P + col0 + (int64_t)u8 * 8;
                            const uint32_t mx = jd.x_dtype == QVB8_BF16 ? amax_x8<QVB8_BF16>(jd.X, off) : amax_x8<QVB8_F32>(jd.X, off);
                            if (mx > 0x477fffffu) atomicMax(&ctl.amax[m], mx);  // only magnitudes of 2^16 and above matter
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctl.amax_ready));
                    mbar_wait(smem_u32(&ctl.amax_ready), 0, abort_flag, 5);
                    if (ctid < M) ctl.kexp[ctid] = (uint8_t)prescale_exp(ctl.amax[ctid]);
                }
                const uint32_t *amax = ctl.amax;
                stage_slice<DUAL, true>(jd.X, jd.x_dtype, jd.P, kc0, NC, M, MP, xs_a, xs_b, cwarp, CWARPS, lane,
                                        [&](int m) { return prescale ? pow2f(-prescale_exp(amax[m])) : 1.f; }, psum_w);
            } else {
                // ---- a later job of this CTA's range (a list's CTA meets one or two jobs per launch, so this is rare):
                // every consumer warp of the CTA meets here -- all have left the previous job, the staged activations
                // may be replaced -- and stages its slice from global memory.
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl.job_done));
                alive = mbar_wait(smem_u32(&ctl.job_done), par(kj - 1), abort_flag, 10);
                // the finishing warps have reached the previous job: they wait on the same once-per-job barriers by
                // parity, so no barrier may complete twice while one of them still waits for the first completion
                if (alive) alive = mbar_wait(smem_u32(&ctl.fin_started), par(kj - 1), abort_flag, 12);
                if (!alive) break;
                const JobDesc &pj = jobs[job - 1];
                if (pj.X == jd.X && pj.P == jd.P && pj.x_dtype == jd.x_dtype && pj.kc0 == jd.kc0 && pj.nc_total == jd.nc_total &&
                    pj.x_mode == jd.x_mode) {
                    // the same activations as the job before (the experts of a mixture layer all read the layer's input):
                    // what is staged stays, the slice's sums move to this job's set
                    const float *prev = psum + (((kj - 1) & 1) * CWARPS + cwarp) * M;
                    for (int m = lane; m < M; m += 32) psum_w[m] = prev[m];
                } else {
                    stage_slice<DUAL, true>(jd.X, jd.x_dtype, jd.P, kc0, NC, M, MP, xs_a, xs_b, cwarp, CWARPS, lane,
                                            [](int) { return 1.f; }, psum_w);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl.x_ready));
            alive = mbar_wait(smem_u32(&ctl.x_ready), par(kj), abort_flag, 5);
            if (!alive) break;
            if (tracer && warp == 0) { if (kj == 0) trace(p.debug, 5); if (kj < 4 && !(p.debug & 64)) trace(p.debug, 16 + 4 * kj); }
            const uint32_t xs_a32 = xvalid ? smem_u32(xs_a) + xoff : smem_u32(zero16);
            const uint32_t xs_b32 = xvalid ? smem_u32(xs_b) + xoff : smem_u32(zero16);
            const __half *xsa = xs_a;

            // ---- walk the run
            for (int i = 0; i < run.nv && alive; ++i, ++vis) {
                const Visit v = run_visit(run, i);
                // the tile's descriptor arrives in a side slot
                const int sslot = vis % NSIDE;
                if (!mbar_wait(side_full0 + 8 * sslot, par(vis / NSIDE), abort_flag, 8)) { alive = false; break; }
                if (tracer && warp == 0 && vis == 0) trace(p.debug, 6);
                const TileDesc *d = reinterpret_cast<const TileDesc *>(side + sslot * side_bytes);
                const int nb = d->nb, cnt = d->cnt;
                const int rb = vis & 1;                                 // hand-over buffer of this visit: free once the finishing
                float *redb = red + rb * RED_FLOATS;                    // warp has taken the sums of the visit before last
                const uint32_t red_full = smem_u32(&pc_.red_full[rb]), red_empty = smem_u32(&pc_.red_empty[rb]);
                const uint32_t red_par = par(vis / 2) ^ 1u;
                float acc[NT][4];
#pragma unroll
                for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
                if (inline_esc) {
                    // ---- in-line escapes.  Lane (g, t) of warp w sums, for rows g and g + 8 and its tokens,
                    // x * (exact - band) over every fourth entry of the row (entries w, w + 4, ... of the tile's list,
                    // those of the visit's columns) and leaves the partial sums for the finishing warp, which adds the four
                    // warps' parts in warp order.  The buffers of this visit's parity are free once the finishing warp has
                    // taken the visit before last.  The code runs with every tile, so it stays warm, unlike the same sums
                    // on the finishing warp; spread over the four warps it delays none of them against the others.
                    if (!mbar_wait(red_empty, red_par, abort_flag, 4)) { alive = false; break; }
                    float *cb = corr + (rb * NW + warp) * (int)(corr_stride_bytes(M) / 4);
                    const EscEntry *ent = reinterpret_cast<const EscEntry *>(side + sslot * side_bytes + DESC_SLOT);
                    const EscEntry *gent = jd.esc_ent + d->esc0;        // the same list in global memory (for the overflow)
                    const int clo = (kc0 + v.sb * cps) * KC, chi = (kc0 + min(v.se * cps, NC)) * KC, cbase = kc0 * KC;
                    if (2 * t < M) {
#pragma unroll
                        for (int hrow = 0; hrow < 2; ++hrow) {
                            const int rs = g + 8 * hrow;
                            float a[NT][2];
#pragma unroll
                            for (int n = 0; n < NT; ++n) a[n][0] = a[n][1] = 0.f;
                            if (d->row[rs] >= 0) {
                                const int ce0 = d->e0[rs], ce1 = d->e1[rs];
                                for (int e = ce0 + ((warp - ce0) & (NW - 1)); e < ce1; e += NW) {
                                    EscEntry en;
                                    if (e < esc_cap) en = ent[e];
                                    else { en.col = __ldg(&gent[e].col); en.delta = __ldg(&gent[e].delta); }
                                    if (en.col >= clo && en.col < chi) {
                                        const int cc = en.col - cbase;
                                        const __half *xp = xsa + ((size_t)slot_of(cc, 2 * t, MP) << 3) + pos_a(cc & 7);
#pragma unroll
                                        for (int n = 0; n < NT; ++n)
#pragma unroll
                                            for (int k = 0; k < 2; ++k)
                                                if (8 * n + 2 * t + k < M)   // consecutive tokens lie four slots (32 halves) apart
                                                    a[n][k] = __fmaf_rn(__half2float(xp[(8 * n + k) * 32]), en.delta, a[n][k]);
                                    }
                                }
                            }
#pragma unroll
                            for (int n = 0; n < NT; ++n)
#pragma unroll
                                for (int k = 0; k < 2; ++k)
                                    if (8 * n + 2 * t + k < M) cb[rs * M + 8 * n + 2 * t + k] = a[n][k];
                        }
                    }
                }
                if (nb == 0) {
                    // per-element class: rows the fragment path cannot read (width outside 3..8, or a row that does not
                    // start on a 16-byte boundary).  One row per warp at a time, ids byte-wise from global memory; the
                    // ring is not used.
                    if (!mbar_wait(red_empty, red_par, abort_flag, 4)) { alive = false; break; }
                    float *rr_out = redb;                               // [16][M] complete row results
                    const int c_lo = v.sb * cps * KC, c_hi = min(v.se * cps, NC) * KC;
                    for (int rr = warp; rr < cnt; rr += NW) {
                        const int q = d->row[rr];
                        const float ms = d->ms[rr], ts = d->ts[rr];
                        const int rnb = __ldg(jd.nbits + q);
                        const int64_t base = __ldg(jd.bit_off + q) + (int64_t)kc0 * KC * rnb;
                        for (int m0 = 0; m0 < M; m0 += 8) {
                            float a[8];
#pragma unroll
                            for (int k = 0; k < 8; ++k) a[k] = 0.f;
                            for (int c = c_lo + lane; c < c_hi; c += 32) {
                                const float wv = band(field_bytes(jd.ids, base + (int64_t)c * rnb, rnb), ts, ms);
#pragma unroll
                                for (int k = 0; k < 8; ++k)
                                    if (m0 + k < M) a[k] = __fmaf_rn(xs_read(xsa, c, m0 + k, MP), wv, a[k]);
                            }
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
#pragma unroll
                                for (int o = 16; o > 0; o >>= 1) a[k] += __shfl_xor_sync(0xffffffffu, a[k], o);
                                if (lane == 0 && m0 + k < M) rr_out[rr * M + m0 + k] = a[k];
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(side_empty0 + 8 * sslot);
                } else {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(side_empty0 + 8 * sslot);    // only the width was needed
                    const uint32_t xbase = (nb >= 6 || !DUAL) ? xs_a32 : xs_b32;
                    bool ok;
#define QV_STREAM(NB_)                                                                                                    \
    ok = cpw == 2 ? stream_tile<NB_, NT, DUAL, 2>(p, ctl.pair_table, abort_flag, rp, NC, v.sb, v.se, warp, lane, xbase, xstep, acc) \
       : cpw == 4 ? stream_tile<NB_, NT, DUAL, 4>(p, ctl.pair_table, abort_flag, rp, NC, v.sb, v.se, warp, lane, xbase, xstep, acc) \
                  : stream_tile<NB_, NT, DUAL, 0>(p, ctl.pair_table, abort_flag, rp, NC, v.sb, v.se, warp, lane, xbase, xstep, acc)
                    switch (nb) {                                       // uniform over the pipe
                        case 7: QV_STREAM(7); break;
                        case 6: QV_STREAM(6); break;
                        case 8: QV_STREAM(8); break;
                        case 5: QV_STREAM(5); break;
                        case 4: QV_STREAM(4); break;
                        default: QV_STREAM(3); break;
                    }
#undef QV_STREAM
                    if (!ok) { alive = false; break; }
                    // hand the partial sums to the finishing warp and go on with the next visit
                    if (!mbar_wait(red_empty, red_par, abort_flag, 4)) { alive = false; break; }
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int k = 0; k < 4; ++k) redb[(warp * 4 * NT + n * 4 + k) * 32 + lane] = acc[n][k];
                }
                if (tracer && warp == 0 && vis == 0) trace(p.debug, 7);
                __syncwarp();
                if (lane == 0) mbar_arrive(red_full);
            }
            if (tracer && warp == 0 && kj < 4 && !(p.debug & 64)) trace(p.debug, 17 + 4 * kj);
        }
        if (tracer && warp == 0) trace(p.debug, 8);
    }
    // ---- several K-ranges (single job): the CTAs (x, 0..S-1) hold partial results of the same tiles; whichever of them
    // gets here last adds the ranges up in range order for all those tiles at once (one ticket per CTA column)
    if (p.S > 1) {
        __threadfence();                                                // this thread's partial results are visible
        __syncthreads();
        __shared__ int last_range;
        if (tid == 0) last_range = atomicAdd(p.ticket + blockIdx.x, 1) == p.S - 1;
        __syncthreads();
        if (last_range) {
            __threadfence();
            const JobDesc &jd = jtab[0];
            int ct0, ct1;
            cta_tiles(jd.ntiles, gridDim.x, blockIdx.x, ct0, ct1);      // (a single job is never rotated)
            const int per_tile = 16 * M;
            const int total = (ct1 - ct0) * per_tile;
            for (int i = tid; i < total; i += blockDim.x) {
                const int tl = ct0 + i / per_tile, rem = i % per_tile;
                const int row = __ldg(&jd.tiles[tl].row[rem / M]), m = rem % M;
                if (row >= 0) {
                    const int64_t o = (int64_t)m * jd.Q + row;
                    float sum = 0.f;
                    for (int r = 0; r < p.S; ++r) sum += __ldcg(p.part + (int64_t)r * M * jd.Q + o);
                    jd.Y[o] = sum;
                }
            }
            if (tid == 0) p.ticket[blockIdx.x] = 0;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// host side

struct Plan {
    int ctas_x, S, nc_per, nc_total, MP, NT, nstg, cps, part_slots, npipe;
    int rs[6], slot_bytes;
    int xs_halves;             // capacity of the staged activations (halves per layout)
    int esc_cap;               // escape entries per side slot
    bool dual;
    size_t smem_bytes;
    int64_t part_bytes, ticket_bytes;
};
constexpr int64_t JOB_TABLE_BYTES_1 = 128;                              // shared-memory job table of a one-job launch
static int64_t psum_bytes_for(int npipe, int64_t M) { return (2 * (int64_t)npipe * NW * M * 4 + 127) / 128 * 128; }

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

// Dynamic shared memory of a CTA: 227 KB per block on this architecture, less two kilobytes for the static part.
constexpr int64_t MAX_DYN_SMEM = 227 * 1024 - 2048;
static_assert(sizeof(Control) <= 2048 - 64, "static shared memory allowance");

// tuning hooks (qvb8_small_m_set_tuning): 0 = choose automatically
static int g_fill_pct = 0, g_force_s = 0, g_force_nstg = 0, g_force_cps = 0, g_debug = 0, g_force_pipes = 0;

static Plan make_plan(int64_t M, int64_t Q, int64_t P, int max_width = 8) {
    Plan pl{};
    pl.nc_total = (int)(P / KC);
    pl.NT = (int)((M + 7) / 8);
    pl.MP = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8 * pl.NT;
    // one CTA per SM, npipe pipes in it.  Two-pipe CTAs (tuning switch) are small enough for the next launch's CTA to sit
    // beside them: back-to-back launches of ONE small shape gain (6144 x 4096 11.5 -> 10.4 us, 4096 x 4096 8.7 -> 7.3 us),
    // but in the layer sequence, where a small launch follows a large one, the whole stack loses (1.89 -> 2.07 ms per
    // token), so four pipes stay the default.
    int npipe = pipes_for(pl.NT);
    if (pl.NT == 1 && npipe == 4 && g_force_pipes == 2) npipe = 2;
    pl.npipe = npipe;
    const int64_t cta_bytes = MAX_DYN_SMEM - 256;                       // dynamic shared memory a CTA may take
    // chunks per stage: long stages mean few, large copies (what the copy engine and HBM like); short K -> short stages
    // (measured for 8 and 16 tokens: short stages win by 16 - 25 % on launches of 10240 rows and more -- more ring
    // slots next to the large staged activations -- and lose 4 - 8 % on 4096 .. 6144 rows; up to 5 tokens long stages win)
    int cps = g_force_cps ? g_force_cps : (pl.nc_total >= 16 && !(M >= 8 && Q >= 8192) ? 8 : 4);
    cps = cps / NW * NW;
    if (cps < NW) cps = NW;
    if (cps > MAX_CPS) cps = MAX_CPS;
    // per pipe next to its ring: side ring, hand-over buffer, escape corrections
    pl.esc_cap = esc_cap_for(P);
    const int64_t pipe_fixed = (int64_t)NSIDE * side_slot_bytes(pl.esc_cap) + (int64_t)2 * NW * 4 * pl.NT * 32 * 4 + corr_bytes(M, pl.esc_cap);
    const int64_t shared_fixed = JOB_TABLE_BYTES_1 + 128 + psum_bytes_for(npipe, M) +
                                 ((XCH_SLOTS + npipe) * 16 * M * 4 + 127) / 128 * 128;   // job table, zeros, activation sums, exchange buffers
    for (;; cps -= NW) {                                                // the longest stage of which two fit per pipe
        pl.cps = cps;
        pl.slot_bytes = 0;                                              // a ring slot: 16 rows of the widest width
        for (int nb = 3; nb <= 8; ++nb) {
            pl.rs[nb - 3] = stage_row_stride(nb, cps);
            if (nb <= max_width && 16 * pl.rs[nb - 3] > pl.slot_bytes) pl.slot_bytes = 16 * pl.rs[nb - 3];
        }
        if (cps <= NW || cta_bytes - shared_fixed - npipe * (pipe_fixed + 2 * (int64_t)pl.slot_bytes) >=
                             (int64_t)KC * pl.MP * 2 * cps)
            break;
    }
    // K-range length: what is left of the CTA's shared memory, after every pipe has a ring of three stages, holds the
    // staged activations.  The second activation layout (no byte permutes for widths 3..5) is staged only when it
    // does not shorten the K-range or the rings.
    const int min_stages = (cps > 8 || npipe > 3) ? 2 : 3;
    const int64_t xs_budget = cta_bytes - shared_fixed - npipe * (pipe_fixed + (int64_t)min_stages * pl.slot_bytes);
    const int64_t xs_one = (int64_t)P * pl.MP * 2;
    pl.dual = pl.MP <= 4 && cta_bytes - shared_fixed - npipe * (pipe_fixed + (int64_t)(min_stages + 1) * pl.slot_bytes) >= 2 * xs_one;
    const int layouts = pl.dual ? 2 : 1;
    int nc_max = xs_budget > 0 ? (int)(xs_budget / (KC * pl.MP * 2 * layouts)) : 0;
    if (nc_max >= cps) nc_max = nc_max / cps * cps;                     // whole stages
    else if (nc_max >= NW) nc_max = nc_max / NW * NW;
    if (nc_max < 1) nc_max = 1;
    const int s_xs = (pl.nc_total + nc_max - 1) / nc_max;
    // one CTA per SM at most; K is split only when the activations of a whole row do not fit
    const int max_tiles = (int)((Q + 15) / 16 + NCLASS - 1);
    int64_t ctas = (int64_t)device_sms() * (g_fill_pct ? g_fill_pct : 100) / 100;
    if (ctas < 1) ctas = 1;
    int S = s_xs;                                                       // the run division balances the pipes by itself
    if (g_force_s) S = g_force_s > s_xs ? g_force_s : s_xs;
    if (S > pl.nc_total) S = pl.nc_total;
    pl.nc_per = (pl.nc_total + S - 1) / S;
    if (pl.nc_per > cps) pl.nc_per = (pl.nc_per + cps - 1) / cps * cps; // K-ranges of whole stages
    if (pl.nc_per > nc_max) pl.nc_per = nc_max;
    pl.S = (pl.nc_total + pl.nc_per - 1) / pl.nc_per;                   // no empty range
    int64_t cx = ctas / pl.S;
    if (cx < 1) cx = 1;
    if (cx > max_tiles) cx = max_tiles;                                 // a CTA takes whole tiles
    pl.ctas_x = (int)cx;
    const int64_t xs_bytes = (int64_t)pl.nc_per * KC * pl.MP * 2 * layouts;
    int nstg = (int)(((cta_bytes - shared_fixed - xs_bytes) / npipe - pipe_fixed) / pl.slot_bytes);
    if (g_force_nstg && g_force_nstg < nstg) nstg = g_force_nstg;
    if (nstg > MAX_STAGES) nstg = MAX_STAGES;
    if (nstg < 2) nstg = 2;
    pl.nstg = nstg;
    pl.smem_bytes = (size_t)(xs_bytes + shared_fixed + npipe * (pipe_fixed + (int64_t)nstg * pl.slot_bytes));
    pl.xs_halves = pl.nc_per * 16 * pl.MP * 8;
    pl.part_slots = pl.S > 1 ? pl.S : 0;                                // partial results only between K-ranges
    pl.part_bytes = ((int64_t)pl.part_slots * M * Q * 4 + 255) / 256 * 256;
    pl.ticket_bytes = pl.S > 1 ? TICKET_BYTES : 0;
    return pl;
}

// Plan of a launch that runs a list of jobs (P and activation element size of every job given): K is never split; one
// buffer holds the staged activations of the job a CTA is in; what is left goes to the copy rings.  Returns false when the list does not fit (activations too large for shared memory next to
// two-stage rings).
constexpr int MIN_RING_CHUNKS = 12;
static bool make_group_plan(int64_t M, const int64_t *Ps, const int *esizes, int njobs, Plan &pl) {
    pl = Plan{};
    pl.NT = (int)((M + 7) / 8);
    pl.MP = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8 * pl.NT;
    const int npipe = pipes_for(pl.NT);
    pl.npipe = npipe;
    pl.dual = false;
    int64_t pmax = 0, pmin = Ps[0];
    for (int j = 0; j < njobs; ++j) {
        if (Ps[j] > pmax) pmax = Ps[j];
        if (Ps[j] < pmin) pmin = Ps[j];
    }
    (void)esizes;
    const int64_t cta_bytes = MAX_DYN_SMEM - 256;
    const int64_t jobs_bytes = job_table_bytes(njobs);
    pl.esc_cap = ESC_CAP_MIN;
    auto pipe_fixed_for = [&](int cap) {
        return (int64_t)NSIDE * side_slot_bytes(cap) + (int64_t)2 * NW * 4 * pl.NT * 32 * 4 + corr_bytes(M, cap);
    };
    int64_t pipe_fixed = pipe_fixed_for(pl.esc_cap);
    const int64_t shared_fixed = jobs_bytes + 128 + psum_bytes_for(npipe, M) + ((XCH_SLOTS + npipe) * 16 * M * 4 + 127) / 128 * 128;
    const int64_t xs_bytes = pmax * pl.MP * 2;
    int cps = g_force_cps ? g_force_cps : (pmin / KC >= 16 ? 8 : 4);
    cps = cps / NW * NW;
    if (cps < NW) cps = NW;
    if (cps > MAX_CPS) cps = MAX_CPS;
    int nstg = 0;
    for (;; cps -= NW) {
        pl.cps = cps;
        pl.slot_bytes = 0;
        for (int nb = 3; nb <= 8; ++nb) {
            pl.rs[nb - 3] = stage_row_stride(nb, cps);
            if (16 * pl.rs[nb - 3] > pl.slot_bytes) pl.slot_bytes = 16 * pl.rs[nb - 3];
        }
        const int64_t room = (cta_bytes - shared_fixed - xs_bytes) / npipe - pipe_fixed;
        nstg = room > 0 ? (int)(room / pl.slot_bytes) : 0;
        // a ring must hold about two long stages' worth of bytes, or the stream stalls at every hiccup of its consumers
        // (measured: with less, a list is slower than the same jobs launched one by one)
        if (nstg * cps >= MIN_RING_CHUNKS || cps <= NW) break;
    }
    if (nstg * cps < MIN_RING_CHUNKS) return false;
    if (g_force_nstg && g_force_nstg < nstg) nstg = g_force_nstg;
    if (nstg > MAX_STAGES) nstg = MAX_STAGES;
    pl.nstg = nstg;
    // escape entries that travel with a tile's descriptor (the in-line escape sums read them from the side slot; what
    // does not fit is read from global memory): as many as the widest job's tiles typically hold, if that costs no
    // ring stage
    for (int cap : {esc_cap_for(pmax) < 256 ? esc_cap_for(pmax) : 256, 128}) {
        if (cap <= pl.esc_cap) continue;
        const int64_t room = (cta_bytes - shared_fixed - xs_bytes) / npipe - pipe_fixed_for(cap);
        if (room >= (int64_t)nstg * pl.slot_bytes) { pl.esc_cap = cap; pipe_fixed = pipe_fixed_for(cap); break; }
    }
    pl.S = 1;
    pl.nc_per = (int)(pmax / KC);
    pl.nc_total = pl.nc_per;
    pl.xs_halves = (int)(pmax / KC) * 16 * pl.MP * 8;
    int64_t ctas = (int64_t)device_sms() * (g_fill_pct ? g_fill_pct : 100) / 100;
    pl.ctas_x = (int)(ctas < 1 ? 1 : ctas);
    pl.smem_bytes = (size_t)(xs_bytes + shared_fixed + npipe * (pipe_fixed + (int64_t)nstg * pl.slot_bytes));
    return true;
}

static bool fast_layout_ok(const qvb8_pack *w, const void *X) {
    return w->P > 0 && w->P % KC == 0 && aligned(w->ids, 16) && aligned(X, 16);
}

template <int NT, bool DUAL, int NPIPE>
static int launch_one(const SmallMParams &prm, const Plan &pl, cudaStream_t st, bool pdl) {
    auto kern = small_m_kernel<NT, DUAL, NPIPE>;
    static thread_local int granted_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != granted_dev) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM) != cudaSuccess)
            return cuda_status("qvb8_small_m: shared memory opt-in");
        granted_dev = dev;
    }
    if (pl.smem_bytes > (size_t)MAX_DYN_SMEM)
        return fail(QVB8_ERR_ARG, "qvb8_small_m: %zu bytes of shared memory needed (tuning out of range)", pl.smem_bytes);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pl.ctas_x, pl.S);
    cfg.blockDim = dim3(NPIPE * PIPE_THREADS);
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, prm) != cudaSuccess) return cuda_status("qvb8_small_m launch");
    return cuda_status("qvb8_small_m launch");
}

static int launch_nt(const SmallMParams &prm, const Plan &pl, cudaStream_t st, bool pdl) {
    switch (pl.NT) {
        case 1:
            if (pl.npipe == 2) return pl.dual ? launch_one<1, true, 2>(prm, pl, st, pdl) : launch_one<1, false, 2>(prm, pl, st, pdl);
            return pl.dual ? launch_one<1, true, pipes_for(1)>(prm, pl, st, pdl) : launch_one<1, false, pipes_for(1)>(prm, pl, st, pdl);
        case 2: return launch_one<2, false, pipes_for(2)>(prm, pl, st, pdl);
        case 3: return launch_one<3, false, pipes_for(3)>(prm, pl, st, pdl);
        case 4: return launch_one<4, false, pipes_for(4)>(prm, pl, st, pdl);
        case 5: return launch_one<5, false, pipes_for(5)>(prm, pl, st, pdl);
        default: return launch_one<6, false, pipes_for(6)>(prm, pl, st, pdl);
    }
}

}  // namespace qv

QV_API void qvb8_small_m_set_tuning(int fill_pct, int force_s, int nstg, int cps, int debug) {
    qv::g_fill_pct = fill_pct > 0 ? fill_pct : 0;
    qv::g_force_s = force_s > 0 ? force_s : 0;
    qv::g_force_nstg = (nstg >= 2 && nstg <= qv::MAX_STAGES) ? nstg : 0;
    qv::g_force_cps = (cps >= qv::NW && cps <= qv::MAX_CPS && cps % qv::NW == 0) ? cps : 0;
    qv::g_debug = debug & 0xff;
    qv::g_force_pipes = (debug >> 8) & 0xf;      // tuning: 2 pipes per CTA for up to 8 tokens instead of 4
}

QV_API int qvb8_debug_trace(unsigned long long *out32) {
    if (!out32) return qv::fail(QVB8_ERR_ARG, "qvb8_debug_trace: null output");
    if (cudaMemcpyFromSymbol(out32, qv::g_trace, sizeof(unsigned long long) * 32) != cudaSuccess)
        return qv::cuda_status("qvb8_debug_trace");
    return QVB8_OK;
}

QV_API int qvb8_device_status(int *status) {
    if (!status) return qv::fail(QVB8_ERR_ARG, "qvb8_device_status: null output");
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, qv::g_error_word, sizeof(int)) != cudaSuccess) return qv::cuda_status("qvb8_device_status");
    if (v == 0)
        if (int rc = qv::prefill_error_word(&v)) return rc;
    if (v == 0)
        if (int rc = qv::peer_error_word(&v)) return rc;
    *status = v;
    return QVB8_OK;
}

QV_API int qvb8_device_status_reset(void) {
    // only the all-reduce's word can be cleared: its waits end by design when a peer is late or gone (the kernel returns
    // and the context stays usable); a wait of the streaming or prefill kernels that gave up means a defect and stays
    return qv::peer_error_reset();
}

QV_API int64_t qvb8_small_m_scratch_bytes(int64_t M, int64_t Q, int64_t P) {
    using namespace qv;
    if (M < 1 || M > MAX_M || Q <= 0 || P <= 0 || P % KC != 0) return 0;
    const Plan pl = make_plan(M, Q, P);
    return pl.part_bytes + pl.ticket_bytes;
}

QV_API int64_t qvb8_plan_bytes(int64_t Q, int64_t n_esc) {
    if (Q < 0 || n_esc < 0) return 0;
    return qv::plan_layout(Q, n_esc).total;
}

QV_API int qvb8_plan_build(const qvb8_pack *w, void *plan, int64_t plan_bytes, void *stream) {
    using namespace qv;
    if (int rc = check_pack(w, "qvb8_plan_build")) return rc;
    if (int rc = check_device("qvb8_plan_build")) return rc;
    if (w->n_esc > 0x7fffffff) return fail(QVB8_ERR_ARG, "qvb8_plan_build: more than 2^31 escapes");
    const PlanLayout L = plan_layout(w->Q, w->n_esc);
    if (!plan || plan_bytes < L.total || !aligned(plan, 16))
        return fail(QVB8_ERR_SCRATCH, "qvb8_plan_build: plan buffer missing, unaligned or smaller than %lld bytes",
                    (long long)L.total);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    uint8_t *base = reinterpret_cast<uint8_t *>(plan);
    int *esc_ptr = reinterpret_cast<int *>(base + L.esc_ptr);
    if (cudaMemsetAsync(base, 0, 256, st) != cudaSuccess ||
        cudaMemsetAsync(base + L.tiles, 0, (size_t)(L.total - L.tiles), st) != cudaSuccess)
        return cuda_status("qvb8_plan_build memset");
    if (w->n_esc > 0) {
        escape_plan_kernel<<<(unsigned)((w->n_esc + 255) / 256), 256, 0, st>>>(
            w->ids, w->min_s, w->tau_s, w->nbits, w->bit_off, w->esc_idx, w->esc_vals, w->n_esc, (int)w->Q, (int)w->P,
            esc_ptr, reinterpret_cast<int *>(base + L.esc_col), reinterpret_cast<float *>(base + L.esc_delta));
        if (int rc = cuda_status("qvb8_plan_build escapes")) return rc;
    }
    if (w->Q > 0) {
        plan_tiles_kernel<<<1, 1024, 0, st>>>(w->nbits, w->bit_off, w->min_s, w->tau_s, w->n_esc > 0 ? esc_ptr : nullptr,
                                              (int)w->Q, L.max_tiles, reinterpret_cast<TileDesc *>(base + L.tiles),
                                              reinterpret_cast<int *>(base));
        if (int rc = cuda_status("qvb8_plan_build tiles")) return rc;
        if (w->n_esc > 0) {
            tile_escapes_kernel<<<1, 1024, 0, st>>>(reinterpret_cast<TileDesc *>(base + L.tiles), reinterpret_cast<int *>(base),
                                                    reinterpret_cast<int *>(base + L.esc_col),
                                                    reinterpret_cast<float *>(base + L.esc_delta),
                                                    reinterpret_cast<EscEntry *>(base + L.esc_ent));
            if (int rc = cuda_status("qvb8_plan_build tile escapes")) return rc;
        }
    }
    return QVB8_OK;
}

namespace qv {
static void fill_job(JobDesc &jd, const qvb8_pack *w, const void *plan, const void *X, float *Y, int x_dtype, int x_mode, int unit0,
                     int prepass = 0) {
    const PlanLayout L = plan_layout(w->Q, w->n_esc);
    const uint8_t *base = reinterpret_cast<const uint8_t *>(plan);
    jd = JobDesc{};
    jd.ids = w->ids; jd.nbits = w->nbits; jd.bit_off = w->bit_off;
    jd.tiles = reinterpret_cast<const TileDesc *>(base + L.tiles);
    jd.ntiles = L.max_tiles;
    jd.esc_ent = w->n_esc > 0 ? reinterpret_cast<const EscEntry *>(base + L.esc_ent) : nullptr;
    jd.X = X; jd.Y = Y;
    jd.Q = (int)w->Q; jd.P = (int)w->P; jd.nc_total = (int)(w->P / KC);
    jd.x_dtype = x_dtype; jd.x_mode = x_mode; jd.unit0 = unit0; jd.yflags = prepass ? 1 : 0;
    jd.kc0 = 0; jd.nsk_part = 0;
}
static void fill_launch(SmallMParams &prm, const Plan &pl, int M) {
    prm.M = M; prm.MP = pl.MP; prm.S = pl.S; prm.nc_per = pl.nc_per; prm.nstg = pl.nstg; prm.debug = g_debug;
    prm.cps = pl.cps; prm.slot_bytes = pl.slot_bytes; prm.esc_cap = pl.esc_cap;
    prm.xs_halves = pl.xs_halves;
    for (int i = 0; i < 6; ++i) prm.rs[i] = pl.rs[i];
    prm.dev_jobs = nullptr; prm.dev_njobs = nullptr; prm.units_per_job = 0;
}

// A list launch whose job table lives in DEVICE memory (written by an earlier kernel of the stream, e.g. from a
// routing decision): up to `cap_jobs` jobs, all with `ntiles` tiles of rows P columns long and no escapes, M <= 8.
// devlist_units: the (tile, stage) units of one such job -- job i of the table must carry unit0 = i * units -- or 0
// when such a list does not fit the kernel (the caller takes another route).
static bool devlist_plan(int64_t M, int64_t P, int cap_jobs, Plan &pl) {
    int64_t Ps[1024];
    int esizes[1024];
    for (int j = 0; j < cap_jobs; ++j) { Ps[j] = P; esizes[j] = 4; }
    return make_group_plan(M, Ps, esizes, cap_jobs, pl);
}
int small_m_devlist_units(int64_t M, int64_t P, int cap_jobs, int ntiles) {
    if (M < 1 || M > 8 || P <= 0 || P % KC != 0 || cap_jobs < 1 || cap_jobs > 1024 || ntiles < 1) return 0;
    Plan pl;
    if (!devlist_plan(M, P, cap_jobs, pl)) return 0;
    const int64_t units = (int64_t)ntiles * ((P / KC + pl.cps - 1) / pl.cps);
    return units * cap_jobs > 0x7fffffff ? 0 : (int)units;
}
int small_m_devlist_launch(const JobDesc *dev_jobs, const int *dev_njobs, int cap_jobs, int64_t M, int64_t P, int ntiles,
                           bool pdl, cudaStream_t st) {
    const int units = small_m_devlist_units(M, P, cap_jobs, ntiles);
    if (units <= 0) return fail(QVB8_ERR_ARG, "qvb8_small_m: a device-resident job list of this shape does not fit");
    Plan pl;
    devlist_plan(M, P, cap_jobs, pl);
    static thread_local SmallMParams prm;
    prm.njobs = cap_jobs;
    prm.units_total = 0;
    prm.ticket = nullptr;
    prm.part = nullptr;
    fill_launch(prm, pl, (int)M);
    prm.dev_jobs = dev_jobs;
    prm.dev_njobs = dev_njobs;
    prm.units_per_job = units;
    return launch_nt(prm, pl, st, pdl);
}
}  // namespace qv

QV_API int qvb8_small_m_ex(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int x_mode, int64_t M,
                           float *Y, void *scratch, int64_t scratch_bytes, int flags, void *stream) {
    using namespace qv;
    if (int rc = check_small_m_args(w, X, x_dtype, x_mode, M, Y, "qvb8_small_m")) return rc;
    if (w->Q == 0) return QVB8_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (plan == nullptr || !fast_layout_ok(w, X) || (w->Q + 15) / 16 + NCLASS - 1 > MAX_TICKET_TILES)
        return launch_small_m_generic(w, X, x_dtype, x_mode, (int)M, Y, st);
    if (!aligned(plan, 16)) return fail(QVB8_ERR_ALIGN, "qvb8_small_m: the plan must be 16-byte aligned");
    const Plan pl = make_plan(M, w->Q, w->P);
    if (pl.part_bytes + pl.ticket_bytes > 0) {
        if (!scratch || scratch_bytes < pl.part_bytes + pl.ticket_bytes)
            return fail(QVB8_ERR_SCRATCH, "qvb8_small_m: scratch of %lld bytes needed, %lld given",
                        (long long)(pl.part_bytes + pl.ticket_bytes), (long long)scratch_bytes);
        if (!aligned(scratch, 16)) return fail(QVB8_ERR_ALIGN, "qvb8_small_m: scratch must be 16-byte aligned");
    }
    static thread_local SmallMParams prm;                               // (a few kilobytes: kept off the stack)
    prm.njobs = 1;
    fill_job(prm.jobs[0], w, plan, X, Y, x_dtype, x_mode, 0);
    prm.ticket = reinterpret_cast<int *>(scratch);
    prm.part = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scratch) + TICKET_BYTES);
    fill_launch(prm, pl, (int)M);
    const bool pdl = (flags & QVB8_FLAG_PDL) != 0;
    return launch_nt(prm, pl, st, pdl);
}

// ---------------------------------------------------------------------------------------------------------------
// several products behind one launch
namespace qv {

// Escape pre-pass of a job list: Y[m, row] = sum over the row's escapes of x[m, col] * (exact - band), for every row of
// every job that has escapes (rows without escapes get 0); the streaming kernel then ADDS its products.  Inside the
// streaming kernel this small, latency-bound sum sits on the finishing warps, which get few issue slots next to the
// warps that stream.  Here it is one THREAD per (tile, row slot) -- a row has a handful of escapes -- so a list of
// dozens of jobs is one resident wave and costs a few dependent memory latencies: fused multiply-adds in stored order
// (same bits every run), entries fetched four at a time so their latencies overlap.
// The activation is narrowed to saturated fp16 first, as the streaming kernel narrows it.
struct EscPrepassParams {
    JobDesc jobs[MAX_JOBS];
    int tile_start[MAX_JOBS + 1];      // first global tile number of job j (jobs without escapes hold no tiles here)
    int njobs, M;
};
__device__ __forceinline__ float prepass_x(const JobDesc &jd, int m, int col) {
    const int64_t i = (int64_t)m * jd.P + col;
    const float x = jd.x_dtype == QVB8_F32 ? load_x<QVB8_F32>(jd.X, i)
                  : jd.x_dtype == QVB8_BF16 ? load_x<QVB8_BF16>(jd.X, i) : load_x<QVB8_F16>(jd.X, i);
    return __half2float(sat_half(x));
}
__global__ void __launch_bounds__(128) escape_prepass_kernel(const __grid_constant__ EscPrepassParams p) {
    // programmatic dependent launch: the streaming kernel that follows may begin its weight prefetch at once; this
    // kernel reads activations and writes outputs only after whatever precedes it in the stream has completed
    pdl_launch_dependents();
    pdl_wait();
    const int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int gt = (int)(gi >> 4), slot = (int)(gi & 15);
    if (gt >= p.tile_start[p.njobs]) return;
    int j = 0;
    while (j + 1 < p.njobs && gt >= p.tile_start[j + 1]) ++j;
    const JobDesc &jd = p.jobs[j];
    const TileDesc *d = jd.tiles + (gt - p.tile_start[j]);
    const int row = __ldg(&d->row[slot]);
    if (row < 0) return;
    const int e0 = __ldg(&d->e0[slot]), e1 = __ldg(&d->e1[slot]);
    const EscEntry *ent = jd.esc_ent + __ldg(&d->esc0);
    for (int m0 = 0; m0 < p.M; m0 += 4) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        for (int e = e0; e < e1; e += 4) {
            int col[4];
            float delta[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int ee = e + k < e1 ? e + k : e1 - 1;
                col[k] = __ldg(&ent[ee].col);
                delta[k] = e + k < e1 ? __ldg(&ent[ee].delta) : 0.f;
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                if (m0 + t < p.M) {
                    float x[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) x[k] = prepass_x(jd, m0 + t, col[k]);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (e + k < e1) s[t] = __fmaf_rn(x[k], delta[k], s[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t)
            if (m0 + t < p.M) jd.Y[(int64_t)(m0 + t) * jd.Q + row] = s[t];
    }
}

// Can this job be part of a list launch?  Through the streaming kernel (plan, layout), activations staged whole.
static bool job_listable(const qvb8_job &jb) {
    return jb.plan && aligned(jb.plan, 16) && fast_layout_ok(jb.w, jb.X) && jb.w->Q > 0 &&
           (jb.w->Q + 15) / 16 + NCLASS - 1 <= MAX_TICKET_TILES &&
           !(jb.x_mode == 1 && jb.x_dtype != QVB8_F16);                  // the prescale pass is the single launch's
}
// K-ranges of a job in a list.  The staged activations of a job take P x MP x 2 bytes of shared memory, which the copy
// rings then lack -- and a list has ONE ring geometry, set by its largest job: one product with many columns and a few
// tokens pushes the whole list to short stages (9B-class stack: 4 tokens x 12288 columns = 96 KB of activations, and
// every job of the list streams with 4-chunk stages, which run a third slower than 8-chunk ones).  So a product whose
// activations exceed XS_BUDGET is cut into KR equal column ranges that run as consecutive jobs of the list: each CTA
// meets the same tiles in every range and every thread adds the later ranges' sums to what it wrote for the first.
// Measured on B200, 16 layers of the 9B-class stack behind one launch: 4 tokens 928 -> 604 us, 8 tokens 1359 -> 919 us
// (a budget of 36-40 KB: 975 us, 20 KB: 1961 us -- every range boundary drains the rings and restages activations).
// Tuning bit 7 switches the cut off; a non-zero force_s of qvb8_small_m_set_tuning also sets this budget, in KB.
constexpr int64_t XS_BUDGET = 72 * 1024;
static int k_ranges(int64_t P, int64_t M) {
    if (g_debug & 128) return 1;
    const int NT = (int)((M + 7) / 8);
    const int64_t MP = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8 * NT;
    const int64_t nc = P / KC;
    const int64_t budget = g_force_s > 0 ? (int64_t)g_force_s * 1024 : XS_BUDGET;   // (force_s doubles as the budget in KB)
    for (int64_t kr = 1; kr <= nc; ++kr)
        if (nc % kr == 0 && (nc / kr) * KC * MP * 2 <= budget) return (int)kr;
    return (int)nc;
}
struct ListEntry { int job, r, kr; };                                   // K-range r of kr of jobs[job]
// Do the entries e[0 .. n) fit one list launch?
static bool list_fits(const qvb8_job *jobs, const ListEntry *e, int n, int64_t M, Plan &pl) {
    int64_t Ps[MAX_JOBS];
    int esizes[MAX_JOBS];
    for (int j = 0; j < n; ++j) {
        Ps[j] = jobs[e[j].job].w->P / e[j].kr;
        esizes[j] = jobs[e[j].job].x_dtype == QVB8_F32 ? 4 : 2;
    }
    return make_group_plan(M, Ps, esizes, n, pl);
}

// Walks the jobs in order and cuts them into list launches: a job (all its K-ranges) joins the open list while it can be
// listed and the list still fits shared memory (at most MAX_JOBS entries); jobs that cannot be listed, and lists of one
// whole job, run as single launches.  on_list(entries, n, plan) / on_single(j) are called in an order that may differ
// from the jobs' order (the jobs are independent).  Returns the first non-zero status of a callback.
template <typename OnList, typename OnSingle>
static int walk_group(const qvb8_job *jobs, int njobs, int64_t M, OnList on_list, OnSingle on_single) {
    ListEntry ent[MAX_JOBS];
    int n = 0;
    Plan pl{};
    auto flush = [&]() -> int {
        int rc = QVB8_OK;
        if (n == 1) rc = on_single(ent[0].job);
        else if (n > 1) rc = on_list(ent, n, pl);
        n = 0;
        return rc;
    };
    for (int j = 0; j < njobs; ++j) {
        if (!job_listable(jobs[j])) {
            if (int rc = on_single(j)) return rc;
            continue;
        }
        const int kr = k_ranges(jobs[j].w->P, M);
        if (kr > MAX_JOBS) {
            if (int rc = on_single(j)) return rc;
            continue;
        }
        Plan trial;
        if (n + kr <= MAX_JOBS) {
            for (int r = 0; r < kr; ++r) ent[n + r] = ListEntry{j, r, kr};
            if (list_fits(jobs, ent, n + kr, M, trial)) {
                pl = trial;
                n += kr;
                continue;
            }
        }
        ListEntry alone[MAX_JOBS];
        for (int r = 0; r < kr; ++r) alone[r] = ListEntry{j, r, kr};
        if (!list_fits(jobs, alone, kr, M, trial)) {                    // fits no list: on its own, the open list stays open
            if (int rc = on_single(j)) return rc;
            continue;
        }
        if (int rc = flush()) return rc;                                // close the open list, start a new one with job j
        for (int r = 0; r < kr; ++r) ent[r] = alone[r];
        pl = trial;
        n = kr;
    }
    return flush();
}
}  // namespace qv

QV_API int64_t qvb8_small_m_group_scratch_bytes(const qvb8_job *jobs, int njobs, int64_t M) {
    using namespace qv;
    if (!jobs || njobs <= 0 || M < 1 || M > MAX_M) return 0;
    for (int j = 0; j < njobs; ++j)
        if (!jobs[j].w || jobs[j].w->P <= 0 || jobs[j].w->Q < 0) return 0;
    int64_t need = 0;
    walk_group(jobs, njobs, M, [](const ListEntry *, int, const Plan &) { return 0; },
               [&](int j) {
                   const int64_t b = qvb8_small_m_scratch_bytes(M, jobs[j].w->Q, jobs[j].w->P);
                   if (b > need) need = b;
                   return 0;
               });
    return need;
}

/* How qvb8_small_m_group would run these jobs (host arithmetic only; nothing is launched, no device needed):
 * list_launches = launches of the streaming kernel that run a list, list_entries = jobs of those lists (a product cut
 * into column ranges counts once per range), single_jobs = jobs that run on their own. */
QV_API int qvb8_small_m_group_describe(const qvb8_job *jobs, int njobs, int64_t M, int *list_launches, int *list_entries,
                                       int *single_jobs) {
    using namespace qv;
    if (!jobs || njobs <= 0 || M < 1 || M > MAX_M || !list_launches || !list_entries || !single_jobs)
        return fail(QVB8_ERR_ARG, "qvb8_small_m_group_describe: bad arguments");
    for (int j = 0; j < njobs; ++j)
        if (!jobs[j].w || jobs[j].w->P <= 0 || jobs[j].w->Q < 0)
            return fail(QVB8_ERR_ARG, "qvb8_small_m_group_describe: job %d has no pack", j);
    int launches = 0, entries = 0, singles = 0;
    walk_group(jobs, njobs, M,
               [&](const ListEntry *, int n, const Plan &) { ++launches; entries += n; return 0; },
               [&](int) { ++singles; return 0; });
    *list_launches = launches;
    *list_entries = entries;
    *single_jobs = singles;
    return QVB8_OK;
}

QV_API int qvb8_small_m_group(const qvb8_job *jobs, int njobs, int64_t M, void *scratch, int64_t scratch_bytes, int flags,
                              void *stream) {
    using namespace qv;
    if (!jobs || njobs <= 0) return fail(QVB8_ERR_ARG, "qvb8_small_m_group: no jobs");
    for (int j = 0; j < njobs; ++j) {
        const qvb8_job &jb = jobs[j];
        if (int rc = check_small_m_args(jb.w, jb.X, jb.x_dtype, jb.x_mode, M, jb.Y, "qvb8_small_m_group")) return rc;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool pdl = (flags & QVB8_FLAG_PDL) != 0;
    auto on_single = [&](int j) -> int {
        const qvb8_job &jb = jobs[j];
        return qvb8_small_m_ex(jb.w, jb.plan, jb.X, jb.x_dtype, jb.x_mode, M, jb.Y, scratch, scratch_bytes, flags, stream);
    };
    auto on_list = [&](const ListEntry *ent, int n, const Plan &pl) -> int {
        static thread_local SmallMParams prm;
        static thread_local EscPrepassParams esc;
        // A list's escapes: a pre-pass kernel leaves the corrections in Y before the streaming kernel adds its sums.  The
        // alternative (tuning bit 5, up to INLINE_ESC_MAX_M tokens): the four consumer warps sum each tile's entries in
        // line, a quarter each -- correct and tested, but measured slower on B200 (9B-class stack, one token, same box:
        // 1.23-1.28 ms against 1.17-1.21 ms with the pre-pass, whose 56 us it saves: the sums sit in front of every
        // tile's stream on all four warps).
        const bool use_prepass = (g_debug & 32) == 0 || M > INLINE_ESC_MAX_M;
        prm.njobs = n;
        esc.njobs = n;
        esc.M = (int)M;
        esc.tile_start[0] = 0;
        int64_t units = 0;
        for (int j = 0; j < n; ++j) {
            const qvb8_job &jb = jobs[ent[j].job];
            JobDesc &jd = prm.jobs[j];
            fill_job(jd, jb.w, jb.plan, jb.X, jb.Y, jb.x_dtype, jb.x_mode, (int)units, jb.w->n_esc > 0 && use_prepass ? 1 : 0);
            if (jb.w->n_esc > 0 && !use_prepass) jd.yflags |= 4;
            const int kr = ent[j].kr, r = ent[j].r;
            const int nc_r = jd.nc_total / kr, nsk_r = (nc_r + pl.cps - 1) / pl.cps;
            jd.nc_total = nc_r;
            jd.kc0 = r * nc_r;
            jd.nsk_part = nsk_r * kr;
            if (r > 0) jd.yflags |= 2;
            // the pre-pass sees a pack once (its first range), with all its columns
            esc.jobs[j] = jd;
            esc.tile_start[j + 1] = esc.tile_start[j] + (jb.w->n_esc > 0 && r == 0 && use_prepass ? jd.ntiles : 0);
            if (r == kr - 1) units += (int64_t)jd.ntiles * jd.nsk_part;
        }
        if (units > 0x7fffffff) return fail(QVB8_ERR_ARG, "qvb8_small_m_group: the list is too long for one launch");
        prm.units_total = (int)units;
        if (esc.tile_start[n] > 0) {                                   // the escapes first: corrections into Y
            const int64_t threads = (int64_t)esc.tile_start[n] * 16;
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3((unsigned)((threads + 127) / 128));
            cfg.blockDim = dim3(128);
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = pdl ? 1 : 0;
            if (cudaLaunchKernelEx(&cfg, escape_prepass_kernel, esc) != cudaSuccess)
                return cuda_status("qvb8_small_m_group escape pre-pass launch");
            if (int rc = cuda_status("qvb8_small_m_group escape pre-pass")) return rc;
        }
        prm.ticket = nullptr;
        prm.part = nullptr;
        fill_launch(prm, pl, (int)M);
        return launch_nt(prm, pl, st, pdl);
    };
    return walk_group(jobs, njobs, M, on_list, on_single);
}

QV_API int qvb8_small_m(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, float *Y, void *scratch,
                        int64_t scratch_bytes, void *stream) {
    return qvb8_small_m_ex(w, nullptr, X, x_dtype, x_mode, M, Y, scratch, scratch_bytes, 0, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// qvb8_small_m_static: the streaming product for callers that cannot hand the library a scratch buffer and cannot
// let it allocate one -- a call made from inside a memory-pool callback, from a thread that must never enter the
// CUDA allocator because another thread holds a capture open, or from a host binding (cgo, JNI) whose runtime gives
// it no device allocator at all.  Their K-range partial results and tile tickets live in a fixed array that is part
// of the loaded module; its address is looked up once per device.
namespace qv {

constexpr int64_t STATIC_SCRATCH_BYTES = 4ll << 20;            // tickets (256 KB) + 3.75 MB of partial results
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_STATIC_DEVICES = 64;
static void *g_static_ptr[MAX_STATIC_DEVICES] = {};

// Address of the array on the current device, looked up once per device.  Nothing is cleared here: a file-scope
// __device__ array is zero when the module is loaded, and every call leaves the ticket area (the only part that must
// start at zero) zero again.  The look-up is a host-side query that touches no stream.
static int static_scratch(void **out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cuda_status("qvb8_small_m_static: current device");
    if (dev < 0 || dev >= MAX_STATIC_DEVICES)
        return fail(QVB8_ERR_ARG, "qvb8_small_m_static: device index %d is beyond the %d this entry point tracks", dev,
                    MAX_STATIC_DEVICES);
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p)
            return cuda_status("qvb8_small_m_static: address of the module's scratch array");
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return QVB8_OK;
}

}  // namespace qv

QV_API int64_t qvb8_small_m_static_max_scratch(void) { return qv::STATIC_SCRATCH_BYTES; }

QV_API int qvb8_small_m_static(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int x_mode, int64_t M,
                               float *Y, int flags, void *stream) {
    using namespace qv;
    if (int rc = check_small_m_args(w, X, x_dtype, x_mode, M, Y, "qvb8_small_m_static")) return rc;
    if (w->Q == 0) return QVB8_OK;
    // scratch is used only by the streaming kernel (same condition as qvb8_small_m_ex): the layout-agnostic kernel
    // that serves every other call needs none, so those calls are never refused for their size
    const bool streaming = plan != nullptr && fast_layout_ok(w, X) &&
                           (w->Q + 15) / 16 + NCLASS - 1 <= MAX_TICKET_TILES;
    const int64_t need = streaming ? qvb8_small_m_scratch_bytes(M, w->Q, w->P) : 0;
    if (need > STATIC_SCRATCH_BYTES)
        return fail(QVB8_ERR_SCRATCH,
                    "qvb8_small_m_static: this product needs %lld bytes of scratch, the built-in array holds %lld; "
                    "use qvb8_small_m_ex with a caller-provided buffer",
                    (long long)need, (long long)STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    return qvb8_small_m_ex(w, plan, X, x_dtype, x_mode, M, Y, scratch, STATIC_SCRATCH_BYTES, flags, stream);
}
