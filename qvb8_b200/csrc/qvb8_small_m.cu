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
// contiguous run of 512 columns (384 - 512 bytes) per stage with a bulk asynchronous copy (cp.async.bulk, completion
// counted on an mbarrier), several stages ahead; the tile's descriptor travels with its first stage.  CTAs are
// persistent: a CTA keeps one K-range (its activations stay staged in shared memory as fp16, in fragment order) and
// walks every (gridDim.x)-th tile, so the copy stream never drains between tiles.
//
// Math.  Four consumer warps each take one 128-column chunk of the stage.  Thread (g = lane / 4, t = lane % 4) owns
// the 32 ids of rows g and g + 8 that start at column 32 t -- exactly nb 32-bit words -- and turns them into the A
// fragments of eight m16n8k16 MMAs.  Two ids are converted per instruction: a funnel shift puts one id in the low
// half-word and one in the high half-word of a register, `(r & mask) | 0x64006400` makes the two fp16 numbers
// 1024 + id * 2^e, and one HFMA2 removes the 1024 and the 2^e exactly.  At the end of a tile the warps hand their
// partial accumulators to a sixth, finishing warp through shared memory and go on streaming; the finishing warp adds
// them in warp order, applies min_s / tau_s, adds the escape corrections it has summed meanwhile (per row, in
// stored order) and writes the result.  K-ranges of one tile are added in range order by whichever CTA finishes the
// tile last (a ticket counter per tile).  Every sum has a fixed order: results are identical from run to run.
//
// Waits.  Every wait on an mbarrier is bounded: after two seconds (or SPIN_LIMIT polls) the waiter raises a per-CTA
// abort flag and a device-wide error word (qvb8_device_status), every other waiter gives up too, and the kernel
// runs to its end with a meaningless result instead of hanging.
#include "common.cuh"

namespace qv {

int launch_fix_escapes(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y, cudaStream_t st);
int launch_small_m_generic(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int M, float *Y,
                           cudaStream_t st);
int check_small_m_args(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, const float *Y,
                       const char *who);

constexpr int KC = 128;                   // columns per chunk
constexpr int NW = 4;                     // consumer warps = chunks per stage
constexpr int PRODUCER_WARP = NW;         // issues the bulk copies
constexpr int FINISHER_WARP = NW + 1;     // escape corrections, cross-warp sums, scaling, output, K-range tickets
constexpr int NTHREADS = (NW + 2) * 32;
constexpr int MAX_STAGES = 8;
constexpr int NCLASS = 7;                 // widths 3..8 -> class 0..5; every other width -> class 6 (per-element path)
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

// One tile of the plan: up to 16 rows of one width.  400 bytes, 16-byte aligned: copied whole by one bulk copy.
struct TileDesc {
    int nb;                 // width of the rows; 0 = per-element class (width outside 3..8 or unaligned row start)
    int cnt;                // real rows (the rest is padding)
    int pad[2];
    int row[16];            // output row, -1 = padding
    uint32_t b16[16];       // byte offset of the row in `ids`, in 16-byte units
    float ms[16], ts[16];   // min_s, tau_s
    int e0[16], e1[16];     // the row's range in the escape plan
};
static_assert(sizeof(TileDesc) == 400, "descriptor size");
constexpr int DESC_BYTES = 400;
constexpr int DESC_SLOT = 416;            // descriptor area of a ring slot

// Plan buffer layout (offsets in bytes, each section 256-byte aligned):
//   [0]  header: int ntiles
//   esc_ptr   int[Q + 1]     first escape of each row
//   esc_col   int[n_esc]     column of each escape
//   esc_delta float[n_esc]   exact value - band value
//   tiles     TileDesc[ceil(Q / 16) + NCLASS - 1]
struct PlanLayout {
    int64_t esc_ptr, esc_col, esc_delta, tiles, total;
    int max_tiles;
};
__host__ __device__ inline int64_t up256(int64_t v) { return (v + 255) / 256 * 256; }
inline PlanLayout plan_layout(int64_t Q, int64_t n_esc) {
    PlanLayout L{};
    L.max_tiles = (int)((Q + 15) / 16 + NCLASS - 1);
    L.esc_ptr = 256;
    L.esc_col = L.esc_ptr + up256((Q + 1) * 4);
    L.esc_delta = L.esc_col + up256(n_esc * 4);
    L.tiles = L.esc_delta + up256(n_esc * 4);
    L.total = L.tiles + up256((int64_t)L.max_tiles * DESC_BYTES);
    return L;
}

// Per-CTA control block in static shared memory.
struct Control {
    float sumx[MAX_M];
    int abort;
    alignas(8) uint64_t full[MAX_STAGES];
    alignas(8) uint64_t empty[MAX_STAGES];
    alignas(8) uint64_t red_full[4];      // the consumer warps' partial sums of a tile are in red[buf]
    alignas(8) uint64_t red_empty[4];     // ... and have been consumed by the finishing warp
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
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    const uint64_t t0 = global_ns();
    for (int i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 7) == 7) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > WAIT_LIMIT_NS) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_error_word, 0, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, code);
}
// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned); completion is counted
// on `bar`.  The destination is this CTA's own shared memory.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32) : "memory"); }

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

// Register holding fp16(id[fa]) in the low half and fp16(id[fa + D]) in the high half, from the nb words W of a
// thread's 32-id block.  All shifts and masks fold to constants after unrolling.
template <int NB>
__device__ __forceinline__ uint32_t pair_reg(const uint32_t (&W)[NB], int fa) {
    constexpr int D = Pairing<NB>::D, E = Pairing<NB>::E;
    constexpr int EL = E > 0 ? E : 0;            // mantissa shift of the low id
    constexpr int EH = E < 0 ? -E : 0;           // mantissa shift of the high id
    static_assert(NB * D == 16 + EH - EL, "pairing does not line the two ids up");
    static_assert(EL + NB <= 10 && EH + NB <= 10, "id does not fit the fp16 mantissa");
    constexpr uint32_t FM = (1u << NB) - 1u;
    constexpr uint32_t MASK = (FM << EL) | (FM << (16 + EH));
    constexpr uint32_t SCALE = h_pow2(EL) | (h_pow2(EH) << 16);
    constexpr uint32_t BIAS = h_neg1024_pow2(EL) | (h_neg1024_pow2(EH) << 16);
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
    if constexpr (EL == 0 && EH == 0) {
        asm("sub.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(r), "r"(0x64006400u));
    } else {
        asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(r), "r"(SCALE), "r"(BIAS));
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

// Bytes between rows of a stage.  The eight chunks of a row lie back to back (a contiguous copy); the stride adds
// one chunk's worth of padding (16 bytes for 8-bit rows) so that the 32 lanes of a warp, which read rows g and
// columns 32 t of ONE chunk, fall on distinct banks.
__host__ __device__ constexpr bool stride_ok(int nb, int rs) {
    return nb == 8 ? (rs / 16) % 8 == 1                  // 16-byte loads, quarter warps (rows 2i, 2i+1)
         : nb == 4 ? (rs / 16) % 8 == 4
         : nb == 6 ? (rs / 8) % 16 == 12                 // 8-byte loads, half warps (rows 4i .. 4i+3)
                   : (rs / 4) % 32 == (4 * nb) % 32;     // 4-byte loads, whole warp
}
__host__ __device__ constexpr int stage_row_stride(int nb) {
    int rs = 16 * nb * NW;
    while (!stride_ok(nb, rs)) rs += 16;
    return rs;
}
constexpr int STAGE_ROW_MAX = stage_row_stride(8) > stage_row_stride(7) ? stage_row_stride(8) : stage_row_stride(7);
constexpr int STAGE_BYTES = 16 * STAGE_ROW_MAX;
static_assert(stage_row_stride(3) <= STAGE_ROW_MAX && stage_row_stride(4) <= STAGE_ROW_MAX &&
              stage_row_stride(5) <= STAGE_ROW_MAX && stage_row_stride(6) <= STAGE_ROW_MAX, "stage row size");

// One 128-column chunk of a 16-row tile of width NB: 8 MMAs per token group.
//   wa, wb   shared addresses of this thread's blocks in rows g and g + 8 of the stage
//   xa       shared address of this thread's first activation slot of the chunk (token 8n + g -> + n * 128 bytes)
//   xstep    bytes between the slots of consecutive 8-column groups (= 4 * MP * 16; 0 for lanes without a token)
//   DUAL     true: a second activation layout exists for widths that pair ids at distance 4 (xa points into it);
//            false: only layout A is staged and those widths rebuild their operands with byte permutes
template <int NB, int NT, bool DUAL>
__device__ __forceinline__ void chunk_mma(uint32_t wa, uint32_t wb, uint32_t xa, uint32_t xstep, float (&acc)[NT][4]) {
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
                         : "r"(xa + i * xstep + n * 128));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // ids of this MMA: D == 2 -> {8i+4h .. 8i+4h+3} paired (f, f+2);  D == 4 -> {8i+2h, +1, +4, +5} paired (f, f+4)
            const int f0 = D == 2 ? 8 * i + 4 * h : 8 * i + 2 * h;
            const uint32_t a0 = pair_reg<NB>(Wa, f0), a2 = pair_reg<NB>(Wa, f0 + 1);
            const uint32_t a1 = pair_reg<NB>(Wb, f0), a3 = pair_reg<NB>(Wb, f0 + 1);
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
// slots are ordered (chunk, group-in-block i, block t, token).  Inside a slot the halves are permuted so that word
// pairs are the B operands directly:  layout A (ids paired at distance 2): x0 x2 x1 x3 x4 x6 x5 x7;
// layout B (distance 4): x0 x4 x1 x5 x2 x6 x3 x7.
__device__ __forceinline__ int slot_of(int c, int m, int MP) {
    const int chunk = c >> 7, t = (c >> 5) & 3, i = (c >> 3) & 3;
    return ((chunk * 4 + i) * 4 + t) * MP + m;
}
__device__ __forceinline__ int pos_a(int e) { return (e & 4) | ((e & 1) << 1) | ((e >> 1) & 1); }
// natural-order read of X[m, c] (c relative to the CTA's first column) from layout A
__device__ __forceinline__ float xs_read(const __half *xs, int c, int m, int MP) {
    return __half2float(xs[(slot_of(c, m, MP) << 3) + pos_a(c & 7)]);
}

template <int XT>
__device__ __forceinline__ void stage_x8(const void *__restrict__ X, int64_t off, uint32_t (&h)[8]) {
    // h[k] = fp16 bits of the k-th activation, saturated
    if constexpr (XT == QVB8_F16) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(X) + off));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { h[2 * k] = w[k] & 0xffffu; h[2 * k + 1] = w[k] >> 16; }
    } else if constexpr (XT == QVB8_BF16) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(X) + off));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            h[2 * k] = __half_as_ushort(sat_half(__uint_as_float(w[k] << 16)));
            h[2 * k + 1] = __half_as_ushort(sat_half(__uint_as_float(w[k] & 0xffff0000u)));
        }
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(X) + off));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(X) + off) + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) h[k] = __half_as_ushort(sat_half(v[k]));
    }
}

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
        const int64_t f = __ldg(esc_idx + i);
        const int q = (int)(f / P), c = (int)(f - (int64_t)q * P);
        const int nb = __ldg(nbits + q);
        const float b = band(field_bytes(ids, __ldg(bit_off + q) + (int64_t)c * nb, nb), __ldg(tau_s + q), __ldg(min_s + q));
        esc_col[i] = c;
        esc_delta[i] = __ldg(esc_vals + i) - b;
        // esc_idx ascends: this escape opens every row after the previous escape's row, up to its own
        const int qprev = i == 0 ? -1 : (int)(__ldg(esc_idx + i - 1) / P);
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
                                                          const int *__restrict__ esc_ptr, int Q, TileDesc *__restrict__ tiles,
                                                          int *__restrict__ header) {
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
}

struct SmallMParams {
    const uint8_t *ids;
    const uint8_t *nbits;      // per-element class only
    const int64_t *bit_off;    // per-element class only
    const TileDesc *tiles;
    const int *ntiles_ptr;     // plan header
    const int *esc_col;        // null: the pack has no escapes
    const float *esc_delta;
    const void *X;
    float *Y;                  // (M, Q)
    float *part;               // (S, M, Q) partial sums when S > 1
    int *ticket;               // one counter per tile when S > 1 (zero on entry, zero on exit)
    int Q, P, M, MP;           // MP: token slots per column group in shared memory (>= M)
    int S;                     // K-ranges (= gridDim.y)
    int nc_per;                // chunks per K-range (the last range may be shorter)
    int nc_total;              // P / 128
    int nstg;                  // slots of the copy ring
    int debug;                 // bit 0: skip the fragment math (copy stream only; tuning experiments)
};

constexpr int SLOT_BYTES = STAGE_BYTES + DESC_SLOT;
constexpr int NRED = 2;                   // hand-over buffers between the consumer warps and the finishing warp

// DUAL: a second activation layout is staged for widths that pair ids at distance 4 (cheap for few tokens).
template <int XT, int NT, bool DUAL>
__global__ void __launch_bounds__(NTHREADS, NT == 1 ? 4 : NT == 2 ? 2 : 1) small_m_kernel(const SmallMParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ Control ctl;
    constexpr int RED_FLOATS = NW * 4 * NT * 32;                       // one hand-over buffer (>= 16 * M floats)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) trace(p.debug, 0);
    const int split = blockIdx.y;
    const int kc0 = split * p.nc_per;                                  // first chunk of this K-range
    const int NC = min(p.nc_per, p.nc_total - kc0);                    // chunks in this K-range (>= 1 by construction)
    const int NSK = (NC + NW - 1) / NW;                                // stages along K per tile
    const int MP = p.MP, M = p.M;
    const int nstg = p.nstg;
    // dynamic shared memory:
    //   [ring: nstg x (16-row stage + descriptor)] [activations A] [activations B] [warp partials x NRED]
    //   [16 zero bytes] [escape corrections]
    const int xs_halves = p.nc_per * 16 * MP * 8;                      // halves per activation layout
    __half *xs_a = reinterpret_cast<__half *>(smem + (size_t)nstg * SLOT_BYTES);
    __half *xs_b = DUAL ? xs_a + xs_halves : xs_a;
    float *red = reinterpret_cast<float *>(xs_a + (DUAL ? 2 : 1) * xs_halves);     // [NRED][NW][4 * NT][32]
    uint32_t *zero16 = reinterpret_cast<uint32_t *>(red + NRED * RED_FLOATS);
    float *corr = reinterpret_cast<float *>(zero16 + 4);               // [16][M], private to the finishing warp
    const bool planned = p.esc_col != nullptr;
    volatile int *abort_flag = &ctl.abort;

    if (tid == 0) {
        for (int s = 0; s < nstg; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 1);
            mbar_init(smem_u32(&ctl.empty[s]), NW);
        }
        for (int b = 0; b < NRED; ++b) {
            mbar_init(smem_u32(&ctl.red_full[b]), NW);
            mbar_init(smem_u32(&ctl.red_empty[b]), 1);
        }
        ctl.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (tid < 4) zero16[tid] = 0u;
    __syncthreads();
    const int ntiles = __ldg(p.ntiles_ptr);
    const int tstep = gridDim.x;
    if (tid == 0) trace(p.debug, 1);

    if (warp == PRODUCER_WARP) {
        // ================= producer warp: lane r copies row r of every stage; lane 16 the tile's descriptor ===========
        int slot = 0;
        uint32_t phase = 0;
        bool alive = true;
        int tile = blockIdx.x;
        int nb = 0, cnt = 0;
        uint32_t b16 = 0;
        auto fetch = [&](int t) {
            if (t < ntiles) {
                nb = __ldg(&p.tiles[t].nb);
                cnt = __ldg(&p.tiles[t].cnt);
                b16 = lane < 16 ? __ldg(&p.tiles[t].b16[lane]) : 0u;
            }
        };
        fetch(tile);
        bool first = true;
        while (tile < ntiles && alive) {
            const int cur = tile, cnb = nb, ccnt = cnt;
            if (first) trace(p.debug, 2);
            const uint8_t *src = p.ids + ((uint64_t)b16 + (uint64_t)kc0 * cnb) * 16u;
            tile += tstep;
            fetch(tile);                                                // next descriptor loads while this tile is issued
            const uint32_t dst_row = (uint32_t)(lane * stage_row_stride(cnb ? cnb : 8));
            const int nstages = cnb ? NSK : 1;
            for (int s = 0; s < nstages; ++s) {
                const int chunks = min(NW, NC - s * NW);
                const uint32_t bytes_row = cnb ? (uint32_t)(chunks * 16 * cnb) : 0u;
                const uint32_t full = smem_u32(&ctl.full[slot]);
                if (!mbar_wait(smem_u32(&ctl.empty[slot]), phase ^ 1u, abort_flag, 1)) { alive = false; break; }
                if (lane == 0) mbar_expect_tx(full, bytes_row * (uint32_t)ccnt + (s == 0 ? (uint32_t)DESC_BYTES : 0u));
                __syncwarp();
                const uint32_t slot32 = smem_u32(smem + (size_t)slot * SLOT_BYTES);
                if (cnb && lane < ccnt) bulk_g2s(slot32 + dst_row, src + (size_t)s * NW * 16 * cnb, bytes_row, full);
                if (s == 0 && lane == 16) bulk_g2s(slot32 + STAGE_BYTES, p.tiles + cur, DESC_BYTES, full);
                if (first) { trace(p.debug, 3); first = false; }
                if (++slot == nstg) { slot = 0; phase ^= 1u; }
            }
        }
    } else if (warp == FINISHER_WARP) {
        // ================= finishing warp: per tile, sums the escape corrections of its rows while the tile streams,
        // then takes the consumer warps' partial sums, scales, corrects and writes the rows =================
        asm volatile("bar.sync 2, %0;\n" ::"n"((NW + 1) * 32) : "memory");     // activations staged, sums ready
        const int g = lane >> 2, t = lane & 3;
        const int clo = kc0 * KC, chi = clo + NC * KC;
        float *out = p.S > 1 ? p.part + (int64_t)split * M * p.Q : p.Y;
        // descriptor fields of the next tile, prefetched: rows g, g+8 (fragment owner) and row `lane` (escapes)
        int nb = 0, frow[2] = {-1, -1}, erow = -1, e0 = 0, e1 = 0;
        float fms[2] = {0.f, 0.f}, fts[2] = {0.f, 0.f};
        auto fetch = [&](int tl) {
            if (tl < ntiles) {
                const TileDesc *d = p.tiles + tl;
                nb = __ldg(&d->nb);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    frow[h] = __ldg(&d->row[g + 8 * h]);
                    fms[h] = __ldg(&d->ms[g + 8 * h]);
                    fts[h] = __ldg(&d->ts[g + 8 * h]);
                }
                if (lane < 16) { erow = __ldg(&d->row[lane]); e0 = __ldg(&d->e0[lane]); e1 = __ldg(&d->e1[lane]); }
            }
        };
        int tile = blockIdx.x, count = 0;
        bool alive = true;
        fetch(tile);
        while (tile < ntiles) {
            const int cur = tile, cnb = nb, crow = lane < 16 ? erow : -1, ce0 = e0, ce1 = e1;
            const int myrow[2] = {frow[0], frow[1]};
            const float myms[2] = {fms[0], fms[1]}, myts[2] = {fts[0], fts[1]};
            tile += tstep;
            fetch(tile);
            // ---- escapes: lane r sums row r's corrections x * (exact - band), in stored order, over this K-range
            if (planned) {
                if (crow >= 0) {
                    float *dst = corr + lane * M;
                    for (int m0 = 0; m0 < M; m0 += 8) {
                        float a[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) a[k] = 0.f;
                        for (int e = ce0; e < ce1; e += 4) {
                            int c[4];
                            float dl[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {                   // four independent loads in flight
                                const bool ok = e + j < ce1;
                                c[j] = ok ? __ldg(p.esc_col + e + j) : -1;
                                dl[j] = ok ? __ldg(p.esc_delta + e + j) : 0.f;
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (c[j] >= clo && c[j] < chi) {
#pragma unroll
                                    for (int k = 0; k < 8; ++k)
                                        if (m0 + k < M) a[k] = __fmaf_rn(xs_read(xs_a, c[j] - clo, m0 + k, MP), dl[j], a[k]);
                                }
                            }
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            if (m0 + k < M) dst[m0 + k] = a[k];
                    }
                }
                __syncwarp();
            }
            if (count == 0) trace(p.debug, 9);
            // ---- the consumer warps' partial sums (or, for a per-element tile, complete row results)
            const int buf = count % NRED;
            if (alive) alive = mbar_wait(smem_u32(&ctl.red_full[buf]), (count / NRED) & 1, abort_flag, 3);
            if (count == 0) trace(p.debug, 10);
            const float *rbuf = red + (size_t)buf * RED_FLOATS;
            float acc[NT][4];
            if (cnb != 0) {
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float v = 0.f;
#pragma unroll
                        for (int w = 0; w < NW; ++w) v += rbuf[(w * 4 * NT + n * 4 + k) * 32 + lane];
                        acc[n][k] = v;
                    }
            }
            // thread holds rows g, g+8 of the tile and tokens 8n+2t, 8n+2t+1
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int m = 8 * n + 2 * t + k;
                        float y = 0.f;
                        if (myrow[hrow] >= 0 && m < M) {
                            // y = tau_s * sum(x * id) + min_s * sum(x)   (per-element rows arrive complete)
                            y = cnb != 0 ? __fmaf_rn(myts[hrow], acc[n][2 * hrow + k], myms[hrow] * ctl.sumx[m])
                                         : rbuf[(g + 8 * hrow) * M + m];
                            if (planned) y += corr[(g + 8 * hrow) * M + m];
                            out[(int64_t)m * p.Q + myrow[hrow]] = y;
                        }
                    }
                }
            }
            __syncwarp();                                               // every lane is done with red[buf] and corr
            if (lane == 0) mbar_arrive(smem_u32(&ctl.red_empty[buf]));
            if (count == 0) trace(p.debug, 11);
            if (p.S > 1) {
                // K-ranges: whichever CTA finishes this tile last adds the partial sums in range order
                __threadfence();
                int last = 0;
                if (lane == 0) last = atomicAdd(p.ticket + cur, 1) == p.S - 1;
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow) {
                        if (myrow[hrow] < 0) continue;
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const int m = 8 * n + 2 * t + k;
                                if (m < M) {
                                    const int64_t o = (int64_t)m * p.Q + myrow[hrow];
                                    float s = 0.f;
                                    for (int r = 0; r < p.S; ++r) s += __ldcg(p.part + (int64_t)r * M * p.Q + o);
                                    p.Y[o] = s;
                                }
                            }
                        }
                    }
                    if (lane == 0) p.ticket[cur] = 0;
                }
            }
            if (count == 0) trace(p.debug, 12);
            ++count;
        }
        trace(p.debug, 13);
    } else {
        // ================= consumer warps =================
        // ---- activations of this K-range as fp16 in fragment order (after the previous kernel in the stream)
        pdl_wait();
        if (warp == 0) trace(p.debug, 4);
        {
            const int groups = NC * 16;                                 // 8-column groups in the range
            const int64_t col0 = (int64_t)kc0 * KC;
            const int total = MP * groups;
            constexpr int UNR = 4;                                      // loads in flight per thread
            for (int base = tid; base < total; base += NW * 32 * UNR) {
                uint32_t h[UNR][8];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int idx = base + u * NW * 32;
                    const int m = idx / groups, u8 = idx - m * groups; // u8: natural 8-column group number
                    if (idx < total && m < M) {
                        stage_x8<XT>(p.X, (int64_t)m * p.P + col0 + (int64_t)u8 * 8, h[u]);
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k) h[u][k] = 0u;
                    }
                }
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int idx = base + u * NW * 32;
                    if (idx >= total) continue;
                    const int m = idx / groups, u8 = idx - m * groups;
                    const int sl = slot_of(u8 * 8, m, MP);
                    *reinterpret_cast<uint4 *>(xs_a + (sl << 3)) = make_uint4(
                        h[u][0] | (h[u][2] << 16), h[u][1] | (h[u][3] << 16), h[u][4] | (h[u][6] << 16), h[u][5] | (h[u][7] << 16));
                    if (DUAL)
                        *reinterpret_cast<uint4 *>(xs_b + (sl << 3)) = make_uint4(
                            h[u][0] | (h[u][4] << 16), h[u][1] | (h[u][5] << 16), h[u][2] | (h[u][6] << 16), h[u][3] | (h[u][7] << 16));
                }
            }
            consumer_sync();
            // per-token sums of the narrowed activations, in a fixed order: thread -> every 128th slot, then a fixed
            // tree over the 128 threads (same bits every run)
            float *psum = red;                                          // 128 floats of the hand-over area, free until the first tile ends
            for (int m = 0; m < M; ++m) {
                float sacc = 0.f;
                for (int j = tid; j < groups; j += NW * 32) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(xs_a + ((size_t)(j * MP + m) << 3));
                    const __half2 *hp = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
                    for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(hp[k]); sacc += f.x; sacc += f.y; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, o);
                if (lane == 0) psum[m * NW + warp] = sacc;
            }
            consumer_sync();
            if (tid < M) {
                float sacc = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w) sacc += psum[tid * NW + w];
                ctl.sumx[tid] = sacc;
            }
            asm volatile("bar.sync 2, %0;\n" ::"n"((NW + 1) * 32) : "memory");     // consumers + finishing warp
        }
        pdl_launch_dependents();
        if (warp == 0) trace(p.debug, 5);

        // ---- walk the tiles
        const int g = lane >> 2, t = lane & 3;
        const bool xvalid = NT > 1 || g < MP;                           // lanes whose token slot exists
        const uint32_t xstep = xvalid ? (uint32_t)(4 * MP * 16) : 0u;   // bytes between consecutive 8-column groups
        const uint32_t xchunk = 4 * xstep;                              // bytes per chunk
        const uint32_t xoff = (uint32_t)((t * MP + g) * 16);
        const uint32_t xs_a32 = xvalid ? smem_u32(xs_a) + xoff : smem_u32(zero16);
        const uint32_t xs_b32 = xvalid ? smem_u32(xs_b) + xoff : smem_u32(zero16);
        const uint32_t ring32 = smem_u32(smem);
        int slot = 0, count = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < ntiles; tile += tstep, ++count) {
            // the tile's first stage carries its descriptor
            if (alive) alive = mbar_wait(smem_u32(&ctl.full[slot]), phase, abort_flag, 2);
            if (warp == 0 && count == 0) trace(p.debug, 6);
            const TileDesc *d = reinterpret_cast<const TileDesc *>(smem + (size_t)slot * SLOT_BYTES + STAGE_BYTES);
            const int nb = alive ? d->nb : 0, cnt = alive ? d->cnt : 0;
            const int buf = count % NRED;
            const uint32_t red_par = ((count / NRED) & 1) ^ 1u;        // the finishing warp has released red[buf]
            float *rbuf = red + (size_t)buf * RED_FLOATS;
            float acc[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
            if (nb == 0) {
                // per-element class: rows the fragment path cannot read (width outside 3..8, or a row that does not
                // start on a 16-byte boundary).  One row per warp at a time, ids byte-wise from global memory; the
                // stage holds only the descriptor.
                if (alive) alive = mbar_wait(smem_u32(&ctl.red_empty[buf]), red_par, abort_flag, 4);
                float *rr_out = rbuf;                                   // [16][M] complete row results
                for (int rr = warp; rr < cnt; rr += NW) {
                    const int q = d->row[rr];
                    const float ms = d->ms[rr], ts = d->ts[rr];
                    const int rnb = __ldg(p.nbits + q);
                    const int64_t base = __ldg(p.bit_off + q) + (int64_t)kc0 * KC * rnb;
                    for (int m0 = 0; m0 < M; m0 += 8) {
                        float a[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) a[k] = 0.f;
                        for (int c = lane; c < NC * KC; c += 32) {
                            const float wv = band(field_bytes(p.ids, base + (int64_t)c * rnb, rnb), ts, ms);
#pragma unroll
                            for (int k = 0; k < 8; ++k)
                                if (m0 + k < M) a[k] = __fmaf_rn(xs_read(xs_a, c, m0 + k, MP), wv, a[k]);
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
                if (lane == 0) mbar_arrive(smem_u32(&ctl.empty[slot]));
                if (++slot == nstg) { slot = 0; phase ^= 1u; }
            } else {
                const int RS = stage_row_stride(nb);
                const uint32_t wa_off = (uint32_t)(g * RS + warp * 16 * nb + t * 4 * nb), wb_off = wa_off + 8 * RS;
                const uint32_t xbase = (nb >= 6 || !DUAL) ? xs_a32 : xs_b32;
                for (int s = 0; s < NSK; ++s) {
                    if (s > 0 && alive) alive = mbar_wait(smem_u32(&ctl.full[slot]), phase, abort_flag, 2);
                    const int chunk = s * NW + warp;
                    if (alive && chunk < NC && !(p.debug & 1)) {
                        const uint32_t stage = ring32 + (uint32_t)slot * SLOT_BYTES;
                        const uint32_t xa = xbase + chunk * xchunk;
                        switch (nb) {                                   // CTA-uniform
                            case 7: chunk_mma<7, NT, DUAL>(stage + wa_off, stage + wb_off, xa, xstep, acc); break;
                            case 6: chunk_mma<6, NT, DUAL>(stage + wa_off, stage + wb_off, xa, xstep, acc); break;
                            case 8: chunk_mma<8, NT, DUAL>(stage + wa_off, stage + wb_off, xa, xstep, acc); break;
                            case 5: chunk_mma<5, NT, DUAL>(stage + wa_off, stage + wb_off, xa, xstep, acc); break;
                            case 4: chunk_mma<4, NT, DUAL>(stage + wa_off, stage + wb_off, xa, xstep, acc); break;
                            case 3: chunk_mma<3, NT, DUAL>(stage + wa_off, stage + wb_off, xa, xstep, acc); break;
                            default: break;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctl.empty[slot]));
                    if (++slot == nstg) { slot = 0; phase ^= 1u; }
                }
                // hand the partial sums to the finishing warp and go on with the next tile
                if (alive) alive = mbar_wait(smem_u32(&ctl.red_empty[buf]), red_par, abort_flag, 4);
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int k = 0; k < 4; ++k) rbuf[(warp * 4 * NT + n * 4 + k) * 32 + lane] = acc[n][k];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl.red_full[buf]));
            if (warp == 0 && count == 0) trace(p.debug, 7);
        }
        if (warp == 0) trace(p.debug, 8);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// host side

struct Plan {
    int ctas_x, S, nc_per, nc_total, MP, NT, nstg;
    bool dual;
    size_t smem_bytes;
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

// tuning hooks (qvb8_small_m_set_tuning): 0 = choose automatically
static int g_fill_pct = 0, g_force_s = 0, g_force_nstg = 0, g_debug = 0;

static Plan make_plan(int64_t M, int64_t Q, int64_t P) {
    Plan pl{};
    pl.nc_total = (int)(P / KC);
    pl.NT = (int)((M + 7) / 8);
    pl.MP = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8 * pl.NT;
    const int per_sm = pl.NT == 1 ? 4 : pl.NT == 2 ? 2 : 1;             // resident CTAs per SM the kernel is built for
    // K-range length: bounded by the shared memory the staged activations may take.  The second activation layout
    // (no byte permutes for widths 3..5) is staged only when it does not shorten the K-range.
    const int xs_budget = pl.NT == 1 ? 16 * 1024 : pl.NT == 2 ? 32 * 1024 : 96 * 1024;
    pl.dual = pl.MP <= 4 && (int64_t)P * pl.MP * 2 * 2 <= xs_budget;
    const int layouts = pl.dual ? 2 : 1;
    int nc_max = xs_budget / (KC * pl.MP * 2 * layouts);
    if (nc_max >= NW) nc_max = nc_max / NW * NW;                        // whole stages
    if (nc_max < 1) nc_max = 1;
    const int s_xs = (pl.nc_total + nc_max - 1) / nc_max;
    // CTAs: one resident wave (persistent CTAs walk the tiles); few tiles -> split K further, down to one stage
    const int max_tiles = (int)((Q + 15) / 16 + NCLASS - 1);
    int64_t slots = (int64_t)per_sm * device_sms() * (g_fill_pct ? g_fill_pct : 100) / 100;
    if (slots < 1) slots = 1;
    const int s_cap = pl.nc_total / NW > 0 ? pl.nc_total / NW : 1;
    int S = s_xs;
    if ((int64_t)max_tiles * S < slots) {
        S = (int)((slots + max_tiles - 1) / max_tiles);
        if (S > s_cap) S = s_cap;
        if (S < s_xs) S = s_xs;
    }
    if (g_force_s) S = g_force_s > s_xs ? g_force_s : s_xs;
    if (S > pl.nc_total) S = pl.nc_total;
    if (max_tiles > MAX_TICKET_TILES) S = s_xs;                         // more tiles than counters: no extra split
    pl.nc_per = (pl.nc_total + S - 1) / S;
    if (pl.nc_per > NW) pl.nc_per = (pl.nc_per + NW - 1) / NW * NW;     // K-ranges of whole stages
    if (pl.nc_per > nc_max) pl.nc_per = nc_max;
    pl.S = (pl.nc_total + pl.nc_per - 1) / pl.nc_per;                   // no empty range
    int64_t cx = slots / pl.S;
    if (cx < 1) cx = 1;
    if (cx > max_tiles) cx = max_tiles;
    pl.ctas_x = (int)cx;
    const size_t xs_bytes = (size_t)pl.nc_per * KC * pl.MP * 2 * layouts;
    const size_t red_bytes = (size_t)NRED * NW * 4 * pl.NT * 32 * 4 + (size_t)16 * M * 4;    // hand-over buffers, corrections
    const size_t per_cta = (size_t)(pl.NT == 1 ? 51 : pl.NT == 2 ? 106 : 216) * 1024;
    int nstg = g_force_nstg ? g_force_nstg : (int)((per_cta - xs_bytes - red_bytes - 64) / SLOT_BYTES);
    if (nstg > MAX_STAGES) nstg = MAX_STAGES;
    if (nstg < 2) nstg = 2;
    pl.nstg = nstg;
    pl.smem_bytes = (size_t)nstg * SLOT_BYTES + xs_bytes + red_bytes + 64;
    pl.part_bytes = pl.S > 1 ? (int64_t)pl.S * M * Q * 4 : 0;
    pl.part_bytes = (pl.part_bytes + 255) / 256 * 256;
    pl.ticket_bytes = pl.S > 1 ? TICKET_BYTES : 0;
    return pl;
}

static bool fast_layout_ok(const qvb8_pack *w, const void *X) {
    return w->P > 0 && w->P % KC == 0 && aligned(w->ids, 16) && aligned(X, 16);
}

template <int XT, int NT, bool DUAL>
static int launch_one(const SmallMParams &prm, const Plan &pl, cudaStream_t st, bool pdl) {
    auto kern = small_m_kernel<XT, NT, DUAL>;
    static thread_local int granted_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != granted_dev) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(222 * 1024)) != cudaSuccess)
            return cuda_status("qvb8_small_m: shared memory opt-in");
        granted_dev = dev;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pl.ctas_x, pl.S);
    cfg.blockDim = dim3(NTHREADS);
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

template <int XT>
static int launch_nt(const SmallMParams &prm, const Plan &pl, cudaStream_t st, bool pdl) {
    switch (pl.NT) {
        case 1: return pl.dual ? launch_one<XT, 1, true>(prm, pl, st, pdl) : launch_one<XT, 1, false>(prm, pl, st, pdl);
        case 2: return launch_one<XT, 2, false>(prm, pl, st, pdl);
        case 3: return launch_one<XT, 3, false>(prm, pl, st, pdl);
        case 4: return launch_one<XT, 4, false>(prm, pl, st, pdl);
        case 5: return launch_one<XT, 5, false>(prm, pl, st, pdl);
        default: return launch_one<XT, 6, false>(prm, pl, st, pdl);
    }
}

}  // namespace qv

QV_API void qvb8_small_m_set_tuning(int fill_pct, int force_s, int nstg, int debug) {
    qv::g_fill_pct = fill_pct > 0 ? fill_pct : 0;
    qv::g_force_s = force_s > 0 ? force_s : 0;
    qv::g_force_nstg = (nstg >= 2 && nstg <= qv::MAX_STAGES) ? nstg : 0;
    qv::g_debug = debug;
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
    *status = v;
    return QVB8_OK;
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
                                              (int)w->Q, reinterpret_cast<TileDesc *>(base + L.tiles),
                                              reinterpret_cast<int *>(base));
        if (int rc = cuda_status("qvb8_plan_build tiles")) return rc;
    }
    return QVB8_OK;
}

QV_API int qvb8_small_m_ex(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int x_mode, int64_t M,
                           float *Y, void *scratch, int64_t scratch_bytes, int flags, void *stream) {
    using namespace qv;
    if (int rc = check_small_m_args(w, X, x_dtype, x_mode, M, Y, "qvb8_small_m")) return rc;
    if (w->Q == 0) return QVB8_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (plan == nullptr || x_mode != 0 || !fast_layout_ok(w, X))
        return launch_small_m_generic(w, X, x_dtype, x_mode, (int)M, Y, st);
    if (!aligned(plan, 16)) return fail(QVB8_ERR_ALIGN, "qvb8_small_m: the plan must be 16-byte aligned");
    const Plan pl = make_plan(M, w->Q, w->P);
    if (pl.part_bytes + pl.ticket_bytes > 0) {
        if (!scratch || scratch_bytes < pl.part_bytes + pl.ticket_bytes)
            return fail(QVB8_ERR_SCRATCH, "qvb8_small_m: scratch of %lld bytes needed, %lld given",
                        (long long)(pl.part_bytes + pl.ticket_bytes), (long long)scratch_bytes);
        if (!aligned(scratch, 16)) return fail(QVB8_ERR_ALIGN, "qvb8_small_m: scratch must be 16-byte aligned");
    }
    const PlanLayout L = plan_layout(w->Q, w->n_esc);
    if (pl.S > 1 && L.max_tiles > MAX_TICKET_TILES)
        return fail(QVB8_ERR_ARG, "qvb8_small_m: %d tiles with a split K-range exceed the %d ticket counters", L.max_tiles,
                    MAX_TICKET_TILES);
    const uint8_t *base = reinterpret_cast<const uint8_t *>(plan);
    SmallMParams prm{};
    prm.ids = w->ids; prm.nbits = w->nbits; prm.bit_off = w->bit_off;
    prm.tiles = reinterpret_cast<const TileDesc *>(base + L.tiles);
    prm.ntiles_ptr = reinterpret_cast<const int *>(base);
    if (w->n_esc > 0) {
        prm.esc_col = reinterpret_cast<const int *>(base + L.esc_col);
        prm.esc_delta = reinterpret_cast<const float *>(base + L.esc_delta);
    }
    prm.X = X; prm.Y = Y;
    prm.ticket = reinterpret_cast<int *>(scratch);
    prm.part = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scratch) + TICKET_BYTES);
    prm.Q = (int)w->Q; prm.P = (int)w->P; prm.M = (int)M; prm.MP = pl.MP; prm.S = pl.S;
    prm.nc_per = pl.nc_per; prm.nc_total = pl.nc_total; prm.nstg = pl.nstg; prm.debug = g_debug;
    const bool pdl = (flags & QVB8_FLAG_PDL) != 0;
    if (x_dtype == QVB8_F16) return launch_nt<QVB8_F16>(prm, pl, st, pdl);
    if (x_dtype == QVB8_BF16) return launch_nt<QVB8_BF16>(prm, pl, st, pdl);
    return launch_nt<QVB8_F32>(prm, pl, st, pdl);
}

QV_API int qvb8_small_m(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, float *Y, void *scratch,
                        int64_t scratch_bytes, void *stream) {
    return qvb8_small_m_ex(w, nullptr, X, x_dtype, x_mode, M, Y, scratch, scratch_bytes, 0, stream);
}
