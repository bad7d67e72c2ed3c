// The plan of a pack: the row ordering and regrouped escapes that qvb8_plan_build writes next to a pack and that the
// streaming and prefill kernels read.
#pragma once
#include "common.cuh"

namespace qv {

constexpr int NCLASS = 7;                 // widths 3..8 -> class 0..5; every other width -> class 6 (per-element path)

// One tile of the plan: up to 16 rows of one width.  400 bytes, 16-byte aligned: copied whole by one bulk copy.
struct TileDesc {
    int nb;                 // width of the rows; 0 = per-element class (width outside 3..8 or unaligned row start)
    int cnt;                // real rows (the rest is padding)
    int esc0;               // first entry of the tile's escapes in the plan's entry list (even: 16-byte aligned)
    int nesc;               // number of entries
    int row[16];            // output row, -1 = padding
    uint32_t b16[16];       // byte offset of the row in `ids`, in 16-byte units
    float ms[16], ts[16];   // min_s, tau_s
    int e0[16], e1[16];     // the row's range within the tile's entries
};
static_assert(sizeof(TileDesc) == 400, "descriptor size");
struct EscEntry { int col; float delta; };   // column, exact value - band value
constexpr int DESC_BYTES = 400;

// Plan buffer layout (offsets in bytes, each section 256-byte aligned):
//   [0]  header: int ntiles
//   esc_ptr   int[Q + 1]     first escape of each row
//   esc_col   int[n_esc]     column of each escape
//   esc_delta float[n_esc]   exact value - band value
//   tiles     TileDesc[ceil(Q / 16) + NCLASS - 1]
//   esc_ent   EscEntry[n_esc + tiles]   the escapes again, grouped by tile (each tile's list padded to an even
//                                       length), so that one contiguous copy brings a tile's escapes
struct PlanLayout {
    int64_t esc_ptr, esc_col, esc_delta, tiles, esc_ent, total;
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
    L.esc_ent = L.tiles + up256((int64_t)L.max_tiles * DESC_BYTES);
    L.total = L.esc_ent + up256((n_esc + L.max_tiles + 2) * 8);
    return L;
}

// One product of a launch: a pack (with its plan), its activations and its output -- or one K-RANGE of such a product:
// columns [kc0 * 128, (kc0 + nc_total) * 128) of every row, the ranges of one pack being consecutive jobs of a list that
// share unit0 and nsk_part, so that every CTA (and every thread of it) meets the same tiles in each of them and adds a
// later range's sums to what it wrote for the earlier ones.
struct JobDesc {
    const uint8_t *ids;
    const uint8_t *nbits;      // per-element class only
    const int64_t *bit_off;    // per-element class only
    const TileDesc *tiles;
    const EscEntry *esc_ent;   // escapes grouped by tile; null: the pack has no escapes
    const void *X;             // (M, P), row 0, column 0
    float *Y;                  // (M, Q)
    int ntiles;                // length of the tile table (real tiles first, then empty ones)
    int Q, P;
    int nc_total;              // 128-column chunks of this job (P / 128, or the K-range's share)
    int x_dtype, x_mode;
    int unit0;                 // list launches: (tile, stage) units of the jobs before this one (before the pack's first range)
    int yflags;                // bit 0: an escape pre-pass has put the pack's corrections into Y (sums are added to them
                               // atomically); bit 1: a later K-range (sums are added to what the earlier ranges wrote)
    int kc0;                   // first chunk of the K-range (0 for a whole product)
    int nsk_part;              // stages per tile over ALL K-ranges of the pack (0: this job's own count)
};
static_assert(sizeof(JobDesc) == 96, "job record layout (host and device agree)");

// qvb8_small_m.cu: list launches of the streaming kernel over a job table in device memory
int small_m_devlist_units(int64_t M, int64_t P, int cap_jobs, int ntiles);
int small_m_devlist_launch(const JobDesc *dev_jobs, const int *dev_njobs, int cap_jobs, int64_t M, int64_t P, int ntiles,
                           bool pdl, cudaStream_t st);

}  // namespace qv
