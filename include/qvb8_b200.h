/*
 * qvb8_b200 -- C ABI of the B200 (sm_100a) kernels for the fused decode-in-matmul over QVB8 / QVB8R weight packs.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, launches on that stream on the CURRENT
 * device and returns a status code; nothing here allocates, synchronises the host or keeps state between calls.
 * A non-zero return leaves a message retrievable with qvb8_last_error() (thread-local).  Preconditions are
 * checked on the host and rejected with a status -- the kernels contain no trap or assert.
 *
 * Each declaration names the entry point of the reference's pybind extensions that it replaces (paths below
 * src/qv_band/ of the reference project).
 */
#ifndef QVB8_B200_H
#define QVB8_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QVB8_OK 0
#define QVB8_ERR_ARG 1      /* a null pointer, a size out of range, an unsupported dtype code            */
#define QVB8_ERR_ALIGN 2    /* a pointer the kernels need aligned is not                                  */
#define QVB8_ERR_SCRATCH 3  /* scratch buffer missing or smaller than the *_scratch_bytes() figure        */
#define QVB8_ERR_CUDA 4     /* the CUDA runtime reported an error at launch                               */
#define QVB8_ERR_DEVICE 5   /* the current device is not compute capability 10.x                          */

/* element type codes for activations and dense outputs */
#define QVB8_F16 0
#define QVB8_BF16 1
#define QVB8_F32 2

/* One QVB8 tensor resident in device memory, exactly the buffers the reference's QVBandLinearV8 holds
 * (formats/qvb8/module.py:87-116).
 *   ids        bit-packed ids, LSB-first, row q starting at bit bit_off[q], each id nbits[q] wide; the
 *              buffer ends with at least 8 readable pad bytes (formats/qvb8/decode.py:303-306)
 *   ids_bytes  size of that buffer INCLUDING the pad
 *   min_s,tau_s   per-row origin and step: value = fma((float)id, tau_s[q], min_s[q])
 *   esc_idx    flat positions q*P+c of the escapes, ascending; esc_vals their exact values              */
typedef struct qvb8_pack {
    const uint8_t *ids;
    int64_t ids_bytes;
    const float *min_s;
    const float *tau_s;
    const uint8_t *nbits;
    const int64_t *bit_off;
    int64_t Q;
    int64_t P;
    const int64_t *esc_idx;
    const float *esc_vals;
    int64_t n_esc;
} qvb8_pack;

/* Message of the last failing call on this thread ("" if none). */
const char *qvb8_last_error(void);

/* Library version string. */
const char *qvb8_version(void);

/* Dense restore W[q, c] = T(fma(id, tau_s, min_s)), one rounding to the output type, escapes narrowed the same
 * way and written over their positions.  out is (Q, P) row-major of out_dtype (QVB8_F16 / QVB8_BF16 / QVB8_F32).
 * Replaces `decode` and `decode_bf16` (formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:651-699, 1711-1727; kernels
 * :535-625); the F32 form is the un-narrowed value the GEMV multiplies (:346-353). */
int qvb8_decode(const qvb8_pack *w, int out_dtype, void *out, void *stream);

/* Row gather: out (n, P) of out_dtype = the restored rows rows[0 .. n) (int64 device array), escapes written over.
 * Replaces QVBandEmbeddingV8._decode_rows and the per-row escape loop of its forward (reference
 * formats/qvb8/embedding.py:92-150); like them it restores with a multiplication and an addition (min_s + id * tau_s),
 * so the table is bit-identical with the reference's.  A row index outside [0, Q) yields a row of zeros. */
int qvb8_embed_rows(const qvb8_pack *w, const int64_t *rows, int64_t n, int out_dtype, void *out, void *stream);

/* Greedy token choice over logits (no counterpart in the reference, which takes torch.argmax of the whole logits; the
 * head itself is a QVBandLinearV8 like any other, run/run_inference.py): best_val[m], best_idx[m] = the largest of
 * Y[m, 0 .. V) (fp32, rows ldy floats apart) and index_base + the LOWEST column that holds it; NaNs are passed over (a
 * row of NaNs gives -inf and index_base).  With the vocabulary split over ranks by output rows each rank reduces its
 * slice of the logits to one pair per token and the ranks exchange 16 bytes per token (qvb8_b200/lm_head.py).
 * scratch: qvb8_argmax_scratch_bytes(M) bytes, 8-byte aligned, contents don't matter.  M <= 65535, V < 2^32 - 1. */
int64_t qvb8_argmax_scratch_bytes(int64_t M);
int qvb8_argmax_rows(const float *Y, int64_t M, int64_t V, int64_t ldy, int64_t index_base, float *best_val,
                     int64_t *best_idx, void *scratch, int64_t scratch_bytes, void *stream);

/* Bytes of scratch qvb8_small_m needs for these sizes (0 is possible).  The scratch must be zero-filled once
 * when it is allocated; the kernel leaves it in a reusable state.  Calls that share one scratch buffer must not
 * overlap on the device. */
int64_t qvb8_small_m_scratch_bytes(int64_t M, int64_t Q, int64_t P);

/* Y[m, q] = sum_c X[m, c] * W[q, c] for 1 <= M <= 48, fp32 result (M, Q), W never materialised.
 *   X        (M, P) row-major of x_dtype
 *   x_mode   0: X is narrowed to saturated fp16 first (|x| > 65504 clamps, NaN kept) -- what every fp16-mode
 *               path of the reference does (qvb8_cuda.cu:761-841, :1082);
 *            1: X keeps its range (an exact power-of-two prescale per token instead of the clamp)
 * The weight is the un-narrowed fp32 band value (or the exact escape value), the contract of the reference's
 * M <= 8 GEMV.  Replaces `forward` for M <= 8, `gemv`, `gemv_multi` (qvb8_cuda.cu:1059-1166, 1416-1512, kernels
 * :306-453, :463-470, :507-533) and `mma_multi` (:2566-2671).  Without a plan (see qvb8_small_m_ex) this entry point
 * runs the layout-agnostic kernel; it needs no scratch then. */
int qvb8_small_m(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, float *Y, void *scratch,
                 int64_t scratch_bytes, void *stream);

/* flags of qvb8_small_m_ex */
#define QVB8_FLAG_PDL 1     /* launch with programmatic stream serialization: the kernel's weight prefetch may overlap
                               the tail of the previous kernel in the stream; everything that depends on earlier
                               work (reading X, writing Y and the scratch) waits for it to complete */

/* Plan of a pack, built once per pack (and per escape table) and then passed to every qvb8_small_m_ex call:
 *   - the rows sorted by width (stable) into 16-row tiles of one width, one 400-byte descriptor per tile
 *     (rows, byte offsets, min_s, tau_s, escape ranges) -- the ordering the reference computes per module for its
 *     tensor-core path (formats/qvb8/module.py:230-277 _mma_order: perm / tile_nb);
 *   - the escape list regrouped by row with the difference (exact value - band value) precomputed -- as the
 *     reference does at load time for its mma path (module.py:279-288 esc_starts) and stores in its qvb8r files
 *     (formats/qvb8r/container.py:10-12 esc_delta).
 * The buffer must be 16-byte aligned and hold qvb8_plan_bytes(Q, n_esc) bytes.  The plan refers to the pack's
 * buffers by offset only; it stays valid while their contents do. */
int64_t qvb8_plan_bytes(int64_t Q, int64_t n_esc);
int qvb8_plan_build(const qvb8_pack *w, void *plan, int64_t plan_bytes, void *stream);

/* qvb8_small_m through the streaming kernel: `plan` from qvb8_plan_build (NULL selects the layout-agnostic
 * kernel), plus launch flags. */
int qvb8_small_m_ex(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int x_mode, int64_t M,
                    float *Y, void *scratch, int64_t scratch_bytes, int flags, void *stream);

/* Several products behind ONE launch (no counterpart in the reference, which launches per linear and hides the launch
 * cost with CUDA graphs, decode/proj_graph.py, decode/layer_graph.py).  The jobs run back to back inside the kernel's
 * persistent CTAs: copy rings, barriers and warp roles carry over from one job to the next, so the stream of weight
 * bytes never drains at a job boundary, and the next job's activations are staged while the current one streams.
 * The jobs must be INDEPENDENT: no job may read what another job of the same call writes (projections that read the
 * outputs of earlier ones go into a later call).  All jobs share M; every job needs its plan.  Any number of jobs: a
 * launch takes up to 128, longer lists become several launches.  A product whose staged activations (P x tokens x 2
 * bytes) would crowd the copy rings is cut into column ranges that run as consecutive jobs of the list; jobs the
 * streaming kernel cannot take at all (no plan, P % 128 != 0, unaligned buffers, x_mode 1 on bf16 / fp32 activations)
 * run on their own exactly as qvb8_small_m_ex would; only those need scratch (qvb8_small_m_group_scratch_bytes,
 * zero-filled once).  Results
 * are deterministic (every sum has a fixed order) and agree with separate calls to rounding: a list is one stream of
 * tiles cut into equal per-CTA ranges, so a tile's fixed-order partial sums may be grouped differently, and the escape
 * corrections of a list are summed by a small pre-pass kernel and the products added to them. */
typedef struct qvb8_job {
    const qvb8_pack *w;
    const void *plan;       /* qvb8_plan_build of w */
    const void *X;          /* (M, w->P) of x_dtype */
    float *Y;               /* (M, w->Q) fp32 */
    int x_dtype, x_mode;    /* as for qvb8_small_m */
} qvb8_job;
int64_t qvb8_small_m_group_scratch_bytes(const qvb8_job *jobs, int njobs, int64_t M);
/* How qvb8_small_m_group would run these jobs (host arithmetic only: nothing is launched, no device is needed):
 * launches of the streaming kernel that run a list, the jobs of those lists (a product cut into column ranges counts
 * once per range), and the jobs that run on their own. */
int qvb8_small_m_group_describe(const qvb8_job *jobs, int njobs, int64_t M, int *list_launches, int *list_entries,
                                int *single_jobs);
int qvb8_small_m_group(const qvb8_job *jobs, int njobs, int64_t M, void *scratch, int64_t scratch_bytes, int flags,
                       void *stream);

/* Tuning hook for tests and sweeps (process-wide; 0 = choose automatically): fill_pct = CTAs launched, in percent of
 * one resident wave; force_s = number of K-ranges (raised to what shared memory requires); nstg = slots of the copy
 * ring (2..8); cps = 128-column chunks per ring stage (4, 8, 12 or 16); debug bit 0 = skip the fragment math (copy
 * stream only), bit 1 = record qvb8_debug_trace stamps, bit 2 = skip the row copies (results meaningless), bit 4 = plain
 * bulk copies without the evict-first hint, bit 5 = list launches of up to 4 tokens sum escapes on the consumer warps instead of by the pre-pass kernel,
 * bit 6 = the stamps follow the finishing warp's visits 4..7 instead of the consumers' jobs, bit 7 = list launches do not cut
 * products with many columns into column ranges (a non-zero force_s is also the activation budget of a range, in KB); bits 8..11 =
 * pipes per CTA for up to 8 tokens (2 instead of the default 4). */
void qvb8_small_m_set_tuning(int fill_pct, int force_s, int nstg, int cps, int debug);

/* Tuning aid: with debug bit 1 set, CTA (0, 0) of the streaming kernel stamps the device nanosecond timer at 14 points
 * of its life into a device array; this copies the 32 slots out.  Synchronises the host. */
int qvb8_debug_trace(unsigned long long *out32);

/* Device-side error word of the current device: 0, or the code of the first bounded wait that gave up inside a
 * kernel of this library (1 = copy ring slot never freed, 2 = copy never landed, 3 / 4 = hand-over between the
 * consumer and finishing warps, 5 / 6 = activation staging, 7 / 8 = descriptor ring, 9 = part of a shared tile,
 * 21..27 = prefill: packed ids never landed, weight slot of tensor memory never freed, raw ring slot never freed,
 * activation stage never freed, weights / activations of a K block never arrived, accumulator never completed;
 * 31 = a peer's flag of an all-reduce never arrived).  Synchronises the host. */
int qvb8_device_status(int *status);
/* Clears code 31 (a late or absent peer is an event a caller may recover from: the all-reduce kernel returned and the
 * context is intact).  Codes of the other kernels mean a defect and are not cleared.  Synchronises the host. */
int qvb8_device_status_reset(void);

/* Same product through the layout-agnostic kernel (any P, any id alignment, widths 1..14).  The library falls
 * back to it by itself when qvb8_small_m's layout preconditions do not hold; exported for tests. */
int qvb8_small_m_generic(const qvb8_pack *w, const void *X, int x_dtype, int x_mode, int64_t M, float *Y,
                         void *stream);

/* ---- prefill: hundreds to thousands of tokens --------------------------------------------------------------------
 * Y (M, Q) fp32 = X (M, P) @ W^T with the weight tiles restored from the packed ids inside the kernel and contracted
 * by tcgen05.mma with the accumulator in tensor memory (replaces the reference's restore-to-HBM + cublasGemmEx path,
 * qvb8_cuda.cu:1542-1671).  P % 64 == 0.  `plan` (qvb8_plan_build) gives the row order and the escapes.
 * scratch: qvb8_prefill_scratch_bytes(M, Q, P) bytes, 256-byte aligned (two fp16 copies of X, its row sums, the
 * list of rows wider than 11 bits). */
int64_t qvb8_prefill_scratch_bytes(int64_t M, int64_t Q, int64_t P);
int qvb8_prefill(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int64_t M, float *Y, void *scratch,
                 int64_t scratch_bytes, void *stream);
/* Tuning aid for sweeps (results are wrong while it is set): 1 = no unpack arithmetic, 2 = no activation copies,
 * 4 = no weight fetch, 8 = no tensor-memory stores, 16 = no MMAs, 48 = no MMAs and plain
 * barrier arrivals instead of commits, 64 = polling waits in the MMA and copy threads; 0 = normal. */
void qvb8_prefill_set_tuning(int debug);

/* ---- all-reduce of the row-parallel projections' partial sums over NVLink peer memory ------------------------------
 * Replaces the library collective at the shard boundary of a linear split across cards (reference
 * formats/qvb8/module.py:126-160 row_subset + the NCCL exchange of run/placement.py).  Every rank allocates one exchange
 * area with qvb8_peer_alloc (qvb8_peer_bytes(world, cap) bytes), hands the 64-byte IPC handle to the other ranks of the
 * node, and maps theirs with qvb8_peer_open.  qvb8_peer_allreduce pushes this rank's `n` partial sums into a slot on
 * every rank (plain peer stores, no multicast), raises a flag there, waits (bounded, status word 31) for the other
 * ranks' flags and adds the slots in rank order: the sums are bit-identical on every rank.  bases[r] = rank r's area as
 * mapped in this process; `epoch` = a zeroed uint32 in this rank's device memory.  All ranks make the same calls in the
 * same order; a call is capturable into a CUDA graph.  flags: QVB8_FLAG_PDL as for qvb8_small_m_ex. */
int64_t qvb8_peer_bytes(int world, int64_t cap_floats);
int qvb8_peer_alloc(int64_t bytes, void **ptr, unsigned char handle[64]);
int qvb8_peer_open(const unsigned char handle[64], void **ptr);
int qvb8_peer_close(void *ptr, int own);
int qvb8_peer_allreduce(void *const *bases, int rank, int world, int64_t cap_floats, void *epoch, const float *partial,
                        float *out, int64_t n, int flags, void *stream);
/* The same with the wait limit as a parameter: wait_ns nanoseconds for the peers' flags (0 = the default two seconds),
 * after which the kernel raises status word 31, sums what it has and returns.  A failure detector uses a short limit. */
int qvb8_peer_allreduce_ex(void *const *bases, int rank, int world, int64_t cap_floats, void *epoch, const float *partial,
                           float *out, int64_t n, int flags, uint64_t wait_ns, void *stream);
/* Every rank of a world on ONE device in one cooperative launch, block r acting as rank r (no counterpart in the
 * reference): bases[r] / epochs[r] / partials[r] / outs[r] are rank r's exchange area, epoch counter, input and output,
 * all in this device's memory.  For machines with fewer GPUs than ranks: separate launches that wait on one another
 * carry no guarantee of running together, the blocks of a cooperative launch do. */
int qvb8_peer_allreduce_local(void *const *bases, int world, int64_t cap_floats, void *const *epochs,
                              const float *const *partials, float *const *outs, int64_t n, uint64_t wait_ns, void *stream);
/* All-gather by the same push protocol, for a linear that is split across cards by output rows only (the reference's
 * row_subset, formats/qvb8/module.py:126-160): out[r * n .. (r + 1) * n) = rank r's part[0 .. n), identical on every
 * rank.  `out` holds world * n floats and does not overlap `part`; n % 4 == 0, n <= cap_floats.  All-gathers and
 * all-reduces may be mixed on one communicator (they share the exchange area and the epoch counter).  wait_ns as for
 * qvb8_peer_allreduce_ex.  qvb8_peer_allgather_local: every rank on one device, as qvb8_peer_allreduce_local. */
int qvb8_peer_allgather(void *const *bases, int rank, int world, int64_t cap_floats, void *epoch, const float *part,
                        float *out, int64_t n, int flags, uint64_t wait_ns, void *stream);
int qvb8_peer_allgather_local(void *const *bases, int world, int64_t cap_floats, void *const *epochs,
                              const float *const *parts, float *const *outs, int64_t n, uint64_t wait_ns, void *stream);

/* ---- mixture-of-experts MLP over stacked expert packs -------------------------------------------------------------
 * Stacked layout of one projection of all E experts (reference formats/qvb8/backends_experts.py:144-196): every
 * expert's bit-packed rows concatenated into ONE buffer (expert segments 16-byte aligned, at least 16 pad bytes after
 * the last row), per-row metadata laid out [expert][row], bit offsets global into `ids`.  No escapes. */
typedef struct qvb8_expert_stack {
    const uint8_t *ids;
    int64_t ids_bytes;
    const float *min_s;      /* [E][Q] */
    const float *tau_s;      /* [E][Q] */
    const uint8_t *nbits;    /* [E][Q] */
    const int64_t *bit_off;  /* [E][Q], bits from the start of ids, byte-aligned rows */
    int64_t Q, P;            /* rows per expert, columns (P % 8 == 0) */
} qvb8_expert_stack;

/* out[t] = sum_j w[t,j] * down_e(act(up_e(x_t))), e = idx[t,j]  (reference qvb8_moe_experts_forward,
 * qvb8_cuda.cu:949-992, and qvb8_moe_experts_relu2_forward, :1002-1058).
 *   act 0: `up` is the gate_up pack (2 I rows: gate rows 0..I-1, up rows I..2I-1), H = silu(gate) * up, I = dn->P
 *   act 1: `up` has I rows, H = relu(up)^2
 * X (M, up->P) of x_dtype is narrowed to saturated fp16 first; idx int64 (M, topk); w fp32 (M, topk);
 * out (M, dn->Q) of x_dtype.  Every distinct selected expert is streamed once for all the tokens that chose it.
 * scratch: qvb8_moe_scratch_bytes(M, topk, E, up->P, up->Q, dn->Q, act) bytes, 256-byte aligned, contents don't matter.
 * A (token, expert) pair whose expert index lies outside [0, E), or whose token names the same expert more than M
 * times, never causes an out-of-range access: the pair contributes ZERO to out[t] (the result stays defined) and is
 * reported by qvb8_moe_bad_index (which synchronises). */
int64_t qvb8_moe_scratch_bytes(int64_t M, int64_t topk, int64_t E, int64_t Pup, int64_t Qup, int64_t Qdn, int act);
int qvb8_moe_experts(const void *X, int x_dtype, int64_t M, const int64_t *idx, const float *w, int64_t topk, int64_t E,
                     const qvb8_expert_stack *up, const qvb8_expert_stack *dn, int act, void *out, void *scratch,
                     int64_t scratch_bytes, void *stream);
/* The same through the streaming kernel when per-expert plans are given and M <= 8 (else exactly qvb8_moe_experts):
 * every distinct selected expert is one job of the small-M streaming kernel (bulk-copy rings, tensor-core sums) with all
 * M tokens as its activations; the job tables are written on the device from the routing.  The hidden activations go
 * through that kernel's fp16 staging, each (expert, token) row scaled by a power of two first so that nothing saturates
 * (undone exactly afterwards): a hidden value carries a relative rounding of 2^-11 that qvb8_moe_experts does not have.
 * Needs up->P and dn->P multiples of 128 and 16-byte aligned stacks; otherwise the plans are ignored.
 * qvb8_moe_plan_bytes(E, Q) / qvb8_moe_plan_build: the plans of one stack (E experts of Q rows), built once; 256-byte
 * aligned device memory owned by the caller.  scratch: as qvb8_moe_scratch_bytes says (it covers both routes).
 * qvb8_moe_streams: 1 when this shape, given plans, runs through the streaming kernel. */
int qvb8_moe_streams(int64_t M, int64_t topk, int64_t E, const qvb8_expert_stack *up, const qvb8_expert_stack *dn);
int64_t qvb8_moe_plan_bytes(int64_t E, int64_t Q);
int qvb8_moe_plan_build(const qvb8_expert_stack *stack, int64_t E, void *plan, int64_t plan_bytes, void *stream);
int qvb8_moe_experts_planned(const void *X, int x_dtype, int64_t M, const int64_t *idx, const float *w, int64_t topk,
                             int64_t E, const qvb8_expert_stack *up, const qvb8_expert_stack *dn, const void *up_plan,
                             const void *dn_plan, int act, void *out, void *scratch, int64_t scratch_bytes, void *stream);
int qvb8_moe_bad_index(const void *scratch, int64_t M, int64_t topk, int64_t E, int64_t Pup, int64_t Qup, int64_t Qdn,
                       int act, int *bad);

/* ---- QVB8R: entropy-coded QVB8 (rANS) ------------------------------------------------------------------------------
 * The arrays a reader builds at load from a .qvb8r file (reference formats/qvb8r/container.py:52-89 runtime_tables,
 * blocks_for; the "core" arguments of every qvb8r_cuda entry point, qvb8r_cuda.cu:322-335).  All device pointers. */
typedef struct qvb8r_pack {
    const uint32_t *words;    /* the word stream followed by at least 2048 zero words (readers fetch ahead) */
    const int64_t *tile_off;  /* [n_tiles + 1] first word of each tile */
    const uint64_t *states;   /* [n_tiles][32] initial rANS states */
    const int64_t *tiles;     /* [n_tiles][3] class, first sorted row, rows */
    int64_t n_tiles;
    const int32_t *blocks;    /* [n_blocks][3] class, first tile, tiles (<= 8): runs of same-class tiles */
    int64_t n_blocks;
    const uint32_t *tab;      /* [K][4096] slot tables: symbol | offset << 11 | (freq - 1) << 22 */
    const int32_t *perm;      /* [Q] sorted row -> original row */
    const float *min_s;       /* [Q] by original row */
    const float *tau_s;       /* [Q] */
    const int32_t *drow;      /* [Q] id = symbol + drow[row] */
    int64_t Q, P;             /* P % 64 == 0 */
} qvb8r_pack;

/* every id, (Q, P) int16 in original row order (reference `ids`, qvb8r_cuda.cu:351-363) */
int qvb8r_ids(const qvb8r_pack *w, int16_t *out, void *stream);
/* dense rows of blocks [b0, b0 + nb): T(fma(id, tau_s, min_s)), out_dtype QVB8_F16 / QVB8_BF16 / QVB8_F32.
 * row_base < 0: each row at its ORIGINAL index of a (Q, P) output; row_base >= 0: at its sorted position - row_base
 * (a block range fills a compact chunk).  (reference `decode`, :272-308, :414-432) */
int qvb8r_decode(const qvb8r_pack *w, int out_dtype, void *out, int64_t b0, int64_t nb, int64_t row_base, void *stream);
/* Y (M, Q) fp32 = X (M, P) @ W^T, 1 <= M <= 16, band part only (escapes: qvb8r_fix_escapes).  round_w_fp16 = 0: fp32
 * band value (reference `gemv` / `multi`, fp32 or bf16 X); 1: band value rounded once to fp16 (reference `tc`, fp16 X). */
int qvb8r_small_m(const qvb8r_pack *w, const void *X, int x_dtype, int64_t M, int round_w_fp16, float *Y, void *stream);
/* Y[m, uq[u]] += sum over e in [ptr[u], ptr[u+1]) of X[m, ec[e]] * ed[e], in stored order (reference `fix_escapes`,
 * :310-320, :434-444): X (M, P) fp32, Y (M, Q) fp32, U outputs that have escapes. */
int qvb8r_fix_escapes(const float *X, const int64_t *uq, const int64_t *ptr, const int64_t *ec, const float *ed, float *Y,
                      int64_t U, int64_t M, int64_t P, int64_t Q, void *stream);

/* Embedding lookup over an entropy-coded table kept in device memory: out (n, P) fp32 = rows rows[0 .. n) (int64 device
 * array), restored as the reference's CPU reader does -- min_s + float(id) * tau_s, multiplication then addition -- and
 * the rows' escapes written over (reference `embed_rows`, qvb8r_cpu.cpp:13-58, which decodes on the host because its
 * target cards are small; a B200 keeps the table in HBM).  inv_perm i32[Q]: original row -> sorted position;
 * row_tile i32[Q]: sorted position -> tile; esc_ptr i64[Q + 1], esc_col i32[], esc_val f32[]: the escapes by row.  The
 * `blocks` field of the pack is not used.  A row index outside [0, Q) yields a row of zeros. */
int qvb8r_embed_rows(const qvb8r_pack *w, const int64_t *rows, int64_t n, const int32_t *inv_perm, const int32_t *row_tile,
                     const int64_t *esc_ptr, const int32_t *esc_col, const float *esc_val, float *out, void *stream);

/* qvb8_small_m_ex without a scratch argument and without any allocation (no counterpart in the reference, whose
 * extension allocates its split-K buffer through torch on every call).  For callers that cannot allocate device
 * memory and have no buffer to pass: code running inside an allocator or memory-pool callback, a thread that must
 * stay out of the CUDA allocator while another thread's stream capture is open, a host binding with no device
 * allocator.  The partial results and tile tickets go to a fixed array inside the loaded module
 * (qvb8_small_m_static_max_scratch() bytes: 4 MiB); a product that needs more (qvb8_small_m_scratch_bytes) is
 * refused with QVB8_ERR_SCRATCH and nothing is launched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current): make that first call before any stream capture that uses this entry point.
 *   - The array is shared by every call on the device and keeps its last contents; only the ticket area must be zero
 *     on entry: it is zero when the module is loaded and every call leaves it zero again.
 *   - Two calls that overlap on the device (different streams) race on the array: serialise them. */
int64_t qvb8_small_m_static_max_scratch(void);
int qvb8_small_m_static(const qvb8_pack *w, const void *plan, const void *X, int x_dtype, int x_mode, int64_t M,
                        float *Y, int flags, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QVB8_B200_H */
