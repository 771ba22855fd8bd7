// Host-side builder of the prefill "panel schedule": the order in which the tcgen05 kernel
// visits the kept tiles of a matrix.  A panel is 16 tile rows whose accumulators share
// tensor memory (for SwiGLU: 8 gate rows and the 8 matching up rows); a chunk is 4 tile
// columns = 64 input features = one 128-byte swizzle row of the activation block.  Inside a
// (panel, chunk) cell tiles are ordered by column then row, and vertically adjacent tiles
// of one column are fused into a "run" that one MMA of N = 16*len covers.
#include <cstdlib>
#include <cstring>
#include <vector>
#include "common.h"

namespace {
constexpr int P = MORTAR_PANEL_ROWS;
constexpr int CC = MORTAR_CHUNK_COLS;

inline int panel_of(int trow, int R, int swiglu, int *local) {
    if (!swiglu) { *local = trow % P; return trow / P; }
    const int F = R / 2, half = P / 2;
    const int u = trow < F ? trow : trow - F;
    *local = (u % half) + (trow < F ? 0 : half);
    return u / half;
}


// One tcgen05.mma of M = 128, K = 16 occupies the tensor pipe for max(kMmaFloorClk, N/2) cycles
// (measured: about 45 cycles up to N = 80, then N/2), and the issuing thread and the barrier
// hand-shakes add a per-instruction cost on top, so two kept tiles a few rows apart are cheaper as
// ONE wider MMA over the rows between them (zero tiles in the gaps) than as two narrow ones.
// cover_column picks, for the kept rows s[l] >= 0 of one tile column of a panel, the set of row
// intervals [lo, hi) with the smallest summed cost max(kMmaFloorClk, 8 * len); ties go to fewer
// zero tiles.  Returns the number of intervals.
#ifdef MORTAR_SCHED_TUNING
static int kMmaFloorClk = 45;   // tuning builds: overridable through MORTAR_SCHED_FLOOR
#else
constexpr int kMmaFloorClk = 45;
#endif

inline int cover_column(const int32_t *s, int *lo, int *hi) {
    // best[i]: cheapest cover of the kept rows among rows [0, i); from[i]: start of the last interval
    // (or -1 when row i-1 is dead and simply skipped)
    long best[P + 1];
    int from[P + 1];
    best[0] = 0; from[0] = -1;
    for (int i = 1; i <= P; ++i) {
        best[i] = -1; from[i] = -1;
        if (s[i - 1] < 0) { best[i] = best[i - 1]; from[i] = -1; continue; }
        for (int j = 0; j < i; ++j) {
            if (s[j] < 0) continue;                       // an interval starts on a kept row
            const int len = i - j;
            int gaps = 0;
            for (int k = j; k < i; ++k) gaps += s[k] < 0;
            const long c = best[j] + (long)(8 * len > kMmaFloorClk ? 8 * len : kMmaFloorClk) * 64 + gaps;
            if (best[i] < 0 || c < best[i]) { best[i] = c; from[i] = j; }
        }
    }
    int n = 0, i = P;
    int rlo[P], rhi[P];
    while (i > 0) {
        if (from[i] < 0) { --i; continue; }
        rlo[n] = from[i]; rhi[n] = i; ++n;
        i = from[i];
    }
    for (int k = 0; k < n; ++k) { lo[k] = rlo[n - 1 - k]; hi[k] = rhi[n - 1 - k]; }
    return n;
}
}  // namespace

// Emits the schedule as a list of steps per panel.  A step is the part of a (panel, chunk)
// cell that fits one B stage of the kernel (at most MORTAR_STEP_TILES tile slots, split at run
// boundaries); empty cells produce no step.  Every step is one contiguous record in step_data:
//   [ header: n_tiles, n_runs, meta, init ][ n_runs x uint16, padded to 8 ][ n_tiles x 64 bytes ]
// A run (one MMA) is 16 bits: first local row | first tile slot << 4 | column in chunk << 10 |
// (length - 1) << 12.  init = 1 when the step's first run is the panel's initialising MMA (all 16
// rows, overwrites the accumulators); every other MMA accumulates.  A tile slot holds 16 row
// words; row word = the row's 16 stored 2-bit values with the even columns in bits 0..15 and the
// odd columns in bits 16..31 (column 2q in bits 2q.., column 2q+1 in bits 16+2q..), the order the
// kernel's shift-free expansion reads; slots of rows without a kept tile hold zero codes.
// meta = chunk index | n_tiles << 14 | n_runs << 20, bit 29 = init, bit 30 set when the step reuses
// the activation chunk of the previous step, bit 31 set when it is the last step on that chunk;
// step_meta repeats it per step.  step_off is in 16-byte units.
// Panels 2s and 2s+1 are executed side by side on one stream of activation chunks, so both
// list exactly the same chunks: a panel without tiles on a chunk its partner uses gets an
// empty step (header only) there.
// kind 0: bf16 schedule as described above.  kind 1: int8 schedule -- the MMA's K is 32, so a slot
// is a PAIR of horizontally adjacent tiles (tile columns 2w, 2w+1; a missing half is zero codes), a
// chunk is 4 such pairs = 128 features, a step holds at most MORTAR_STEP_SLOTS_I8 slots, and a
// slot's codes are stored one nibble per code (16 rows x 4 words; word k = columns 8k..8k+7 of the
// pair, stored value = code + 1), the form the kernel's byte-permute expansion reads.
static int build(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes, int32_t R,
                 int32_t C, int32_t swiglu, int32_t kind, int64_t *n_tiles_out, int64_t *n_runs_out,
                 int64_t *n_steps_out, int32_t *n_panels_out, int64_t *data_units_out,
                 uint8_t *step_data, uint32_t *step_off, uint32_t *step_meta,
                 int32_t *panel_step_ptr, uint32_t *panel_mask) {
    if (!row_ptr || !n_tiles_out || !n_runs_out || !n_steps_out || !n_panels_out || !data_units_out)
        return MORTAR_ERR_NULL;
    if (R <= 0 || C <= 0 || C > 65534) return MORTAR_ERR_SHAPE;
    if (swiglu && (R % 2)) return MORTAR_ERR_SHAPE;
    const int units = swiglu ? R / 2 : R;
    const int per_panel = swiglu ? P / 2 : P;
    // panels are executed in pairs: pad to an even count with an all-empty panel
    const int NP = ((units + per_panel - 1) / per_panel + 1) & ~1;
    if (kind != 0 && kind != 1) return MORTAR_ERR_DTYPE;
    const int CW = kind ? (C + 1) / 2 : C;          // columns in slot units
    const int NC = (CW + CC - 1) / CC;
    const int step_cap = kind ? MORTAR_STEP_SLOTS_I8 : MORTAR_STEP_TILES;
    const bool fill = step_data != nullptr;
#ifdef MORTAR_SCHED_TUNING
    if (const char *e = getenv("MORTAR_SCHED_FLOOR")) kMmaFloorClk = atoi(e);
#endif
    if (fill && (!step_off || !step_meta || !panel_step_ptr || !panel_mask || !col_idx || !codes))
        return MORTAR_ERR_NULL;
    // bucket tiles by cell: slot[cell][col_local][row_local] = tile index or -1
    const int64_t cells = (int64_t)NP * NC;
    std::vector<int32_t> slot((size_t)cells * CC * P, -1);
    std::vector<int32_t> slot_b(kind ? (size_t)cells * CC * P : 0, -1);      // right half of a pair (kind 1)
    for (int r = 0; r < R; ++r) {
        if (row_ptr[r + 1] < row_ptr[r]) return MORTAR_ERR_ROWPTR;
        int local;
        const int panel = panel_of(r, R, swiglu, &local);
        for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
            const int c = col_idx ? col_idx[j] : 0;
            if (c >= C) return MORTAR_ERR_COLIDX;
            const int cw = kind ? c / 2 : c;
            const size_t at = (((size_t)panel * NC + cw / CC) * CC + cw % CC) * P + local;
            if (kind && (c & 1)) slot_b[at] = (int32_t)j;
            else slot[at] = (int32_t)j;
        }
    }
    // liveness of a slot: either half of the pair holds a tile; -2 marks "right half only"
    if (kind)
        for (size_t i = 0; i < slot.size(); ++i)
            if (slot[i] < 0 && slot_b[i] >= 0) slot[i] = -2;
    auto live = [&](int32_t v) { return v >= 0 || v == -2; };
    struct Run { int cl, lo, first, len; };
    int64_t nt = 0, nr = 0, ns = 0, units16 = 0, n_gap = 0;
    std::vector<Run> step_runs;
    std::vector<int32_t> step_tiles;           // kind 0: tile index or -1; kind 1: position in `slot` or -1
    const int slot_units = kind ? 16 : 4;      // 16-byte units of codes per slot
    bool step_init = false;            // the step under construction starts with the initialising MMA
    auto flush = [&](int ch, bool reuse, bool last) {
        const int ntile = (int)step_tiles.size(), nrun = (int)step_runs.size();
        const int run_units = (nrun + 7) / 8;
        if (fill) {
            step_off[ns] = (uint32_t)units16;
            const uint32_t meta = (uint32_t)ch | ((uint32_t)ntile << 14) | ((uint32_t)nrun << 20) |
                                  (step_init ? 0x20000000u : 0u) | (reuse ? 0x40000000u : 0u) |
                                  (last ? 0x80000000u : 0u);
            step_meta[ns] = meta;
            uint32_t *hdr = reinterpret_cast<uint32_t *>(step_data + units16 * 16);
            hdr[0] = (uint32_t)ntile; hdr[1] = (uint32_t)nrun; hdr[2] = meta; hdr[3] = step_init ? 1u : 0u;
            uint16_t *rr = reinterpret_cast<uint16_t *>(hdr + 4);
            for (int i = 0; i < run_units * 8; ++i) rr[i] = 0;
            for (int i = 0; i < nrun; ++i)
                rr[i] = (uint16_t)(step_runs[i].lo | (step_runs[i].first << 4) | (step_runs[i].cl << 10) |
                                   ((step_runs[i].len - 1) << 12));
            uint32_t *td = reinterpret_cast<uint32_t *>(step_data + (units16 + 1 + run_units) * 16);
            for (int i = 0; kind && i < ntile; ++i) {
                const int32_t pos = step_tiles[i];
                const int32_t ta = pos >= 0 ? slot[pos] : -1, tb = pos >= 0 ? slot_b[pos] : -1;
                for (int row = 0; row < 16; ++row) {
                    uint32_t ca = 0x55555555u, cb = 0x55555555u;      // stored value 1 = code 0
                    if (ta >= 0) memcpy(&ca, codes + (int64_t)ta * 64 + row * 4, 4);
                    if (tb >= 0) memcpy(&cb, codes + (int64_t)tb * 64 + row * 4, 4);
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t src = k < 2 ? ca : cb;
                        uint32_t w = 0;
                        for (int e = 0; e < 8; ++e) w |= ((src >> (2 * ((k & 1) * 8 + e))) & 3u) << (4 * e);
                        td[(i * 16 + row) * 4 + k] = w;
                    }
                }
            }
            for (int i = 0; !kind && i < ntile; ++i) {
                for (int row = 0; row < 16; ++row) {
                    uint32_t canon = 0x55555555u;                        // stored value 1 = code 0
                    if (step_tiles[i] >= 0) memcpy(&canon, codes + (int64_t)step_tiles[i] * 64 + row * 4, 4);
                    uint32_t w = 0;
                    for (int q = 0; q < 8; ++q) {
                        w |= ((canon >> (4 * q)) & 3u) << (2 * q);
                        w |= ((canon >> (4 * q + 2)) & 3u) << (16 + 2 * q);
                    }
                    td[i * 16 + row] = w;
                }
            }
        }
        units16 += 1 + run_units + slot_units * (int64_t)ntile;
        nt += ntile; nr += nrun; ++ns;
        step_runs.clear(); step_tiles.clear();
        step_init = false;
    };
    // which cells hold at least one tile
    std::vector<uint8_t> cell_used((size_t)cells, 0);
    for (size_t i = 0; i < slot.size(); ++i)
        if (live(slot[i])) cell_used[i / ((size_t)CC * P)] = 1;
    for (int p = 0; p < NP; ++p) {
        uint32_t touched = 0;
        bool initialised = false;       // the panel's accumulators hold defined values
        if (fill) panel_step_ptr[p] = (int32_t)ns;
        const int partner = p ^ 1;      // the kernel runs panels 2s and 2s+1 side by side on shared chunks
        for (int ch = 0; ch < NC; ++ch) {
            const size_t cell = (size_t)p * NC + ch;
            if (!cell_used[cell]) {
                // the partner uses this chunk: emit an empty step so both walk the same chunk list
                if (partner < NP && cell_used[(size_t)partner * NC + ch]) flush(ch, false, true);
                continue;
            }
            bool first_of_chunk = true;
            for (int cl = 0; cl < CC; ++cl) {
                const int32_t *s = &slot[(cell * CC + cl) * P];
                int n_live = 0;
                int32_t lv[P];                                           // >= 0 where the slot is live
                for (int l = 0; l < P; ++l) { lv[l] = live(s[l]) ? 0 : -1; n_live += lv[l] >= 0; }
                if (n_live == 0) continue;
                // intervals [lo, hi) of local rows that one MMA each will cover
                int lo[P], hi[P], n_iv = 0;
                if (!initialised) {
                    // the panel's first MMA overwrites all 256 accumulator columns (dead rows get
                    // zero tiles), so every later MMA of the item accumulates
                    lo[0] = 0; hi[0] = P; n_iv = 1;
                } else {
                    n_iv = cover_column(lv, lo, hi);
                }
                for (int v = 0; v < n_iv; ++v) {
                    const int len = hi[v] - lo[v];
                    if ((int)step_tiles.size() + len > step_cap) {
                        flush(ch, !first_of_chunk, false);
                        first_of_chunk = false;
                    }
                    Run run;
                    run.cl = cl; run.lo = lo[v];
                    run.first = (int)step_tiles.size();
                    run.len = len;
                    if (!initialised) step_init = true;      // always the first run of a fresh step (see below)
                    step_runs.push_back(run);
                    for (int k = lo[v]; k < hi[v]; ++k) {
                        if (kind) step_tiles.push_back(live(s[k]) ? (int32_t)((cell * CC + cl) * P + k) : -1);
                        else step_tiles.push_back(s[k]);                 // -1 = zero tile (gap)
                        if (live(s[k])) touched |= 1u << k;
                        else ++n_gap;
                    }
                    initialised = true;
                }
            }
            if (!step_tiles.empty()) flush(ch, !first_of_chunk, true);
        }
        if (fill) panel_mask[p] = touched;
    }
    if (nt > INT32_MAX || nr > INT32_MAX || ns > INT32_MAX || units16 > 0xffffffffLL) return MORTAR_ERR_CAPACITY;
    if (fill) { panel_step_ptr[NP] = (int32_t)ns; step_off[ns] = (uint32_t)units16; }
    *n_tiles_out = nt; *n_runs_out = nr; *n_steps_out = ns; *n_panels_out = NP; *data_units_out = units16;
    return MORTAR_OK;
}

extern "C" int mortar_sched_sizes(const int32_t *row_ptr, const uint16_t *col_idx, int32_t R, int32_t C,
                                  int32_t swiglu, int64_t *n_tiles, int64_t *n_runs, int64_t *n_steps,
                                  int32_t *n_panels, int64_t *data_units) {
    return build(row_ptr, col_idx, nullptr, R, C, swiglu, 0, n_tiles, n_runs, n_steps, n_panels, data_units,
                 nullptr, nullptr, nullptr, nullptr, nullptr);
}

extern "C" int mortar_build_sched(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes,
                                  int32_t R, int32_t C, int64_t nnz, int32_t swiglu, uint8_t *step_data,
                                  uint32_t *step_off, uint32_t *step_meta, int32_t *panel_step_ptr,
                                  uint32_t *panel_mask) {
    int v = mortar_validate_bcsr(row_ptr, col_idx, codes, R, C, nnz);
    if (v != MORTAR_OK) return v;
    if (!step_data) return MORTAR_ERR_NULL;
    int64_t nt, nr, ns, du; int32_t np;
    return build(row_ptr, col_idx, codes, R, C, swiglu, 0, &nt, &nr, &ns, &np, &du, step_data, step_off,
                 step_meta, panel_step_ptr, panel_mask);
}

extern "C" int mortar_sched_sizes_i8(const int32_t *row_ptr, const uint16_t *col_idx, int32_t R, int32_t C,
                                     int32_t swiglu, int64_t *n_tiles, int64_t *n_runs, int64_t *n_steps,
                                     int32_t *n_panels, int64_t *data_units) {
    return build(row_ptr, col_idx, nullptr, R, C, swiglu, 1, n_tiles, n_runs, n_steps, n_panels, data_units,
                 nullptr, nullptr, nullptr, nullptr, nullptr);
}

extern "C" int mortar_build_sched_i8(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes,
                                     int32_t R, int32_t C, int64_t nnz, int32_t swiglu, uint8_t *step_data,
                                     uint32_t *step_off, uint32_t *step_meta, int32_t *panel_step_ptr,
                                     uint32_t *panel_mask) {
    int v = mortar_validate_bcsr(row_ptr, col_idx, codes, R, C, nnz);
    if (v != MORTAR_OK) return v;
    if (!step_data) return MORTAR_ERR_NULL;
    int64_t nt, nr, ns, du; int32_t np;
    return build(row_ptr, col_idx, codes, R, C, swiglu, 1, &nt, &nr, &ns, &np, &du, step_data, step_off,
                 step_meta, panel_step_ptr, panel_mask);
}
