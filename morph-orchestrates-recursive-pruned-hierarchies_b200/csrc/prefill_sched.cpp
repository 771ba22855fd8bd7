// Host-side builder of the prefill "panel schedule": the order in which the tcgen05 kernel
// visits the kept tiles of a matrix.  A panel is 16 tile rows whose accumulators share
// tensor memory (for SwiGLU: 8 gate rows and the 8 matching up rows); a chunk is 4 tile
// columns = 64 input features = one 128-byte swizzle row of the activation block.  Inside a
// (panel, chunk) cell tiles are ordered by column then row, and vertically adjacent tiles
// of one column are fused into a "run" that one MMA of N = 16*len covers.
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

inline uint32_t idesc_for(int n) {
    // kind::f16, D fp32 (bit 4), A bf16 (bit 7), B bf16 (bit 10), both K-major, N>>3 at 17, M>>4 at 24
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}
}  // namespace

// Emits the schedule as a list of steps per panel.  A step is the part of a (panel, chunk)
// cell that fits one B stage of the kernel (at most MORTAR_STEP_TILES tiles, split at run
// boundaries); empty cells produce no step.  Every step is one contiguous record in
// step_data so a single bulk copy stages it:
//   [ header: n_tiles, n_runs, meta, 0 ][ n_runs run records of 16 bytes ][ n_tiles x 64 bytes ]
// meta = chunk index, bit 30 set when the step reuses the activation chunk of the previous
// step, bit 31 set when it is the last step on that chunk.  step_off is in 16-byte units.
// Panels 2s and 2s+1 are executed side by side on one stream of activation chunks, so both
// list exactly the same chunks: a panel without tiles on a chunk its partner uses gets an
// empty step (header only) there.
static int build(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes, int32_t R,
                 int32_t C, int32_t swiglu, int64_t *n_tiles_out, int64_t *n_runs_out,
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
    const int NC = (C + CC - 1) / CC;
    const bool fill = step_data != nullptr;
    if (fill && (!step_off || !step_meta || !panel_step_ptr || !panel_mask || !col_idx || !codes))
        return MORTAR_ERR_NULL;
    // bucket tiles by cell: slot[cell][col_local][row_local] = tile index or -1
    const int64_t cells = (int64_t)NP * NC;
    std::vector<int32_t> slot((size_t)cells * CC * P, -1);
    for (int r = 0; r < R; ++r) {
        if (row_ptr[r + 1] < row_ptr[r]) return MORTAR_ERR_ROWPTR;
        int local;
        const int panel = panel_of(r, R, swiglu, &local);
        for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
            const int c = col_idx ? col_idx[j] : 0;
            if (c >= C) return MORTAR_ERR_COLIDX;
            slot[(((size_t)panel * NC + c / CC) * CC + c % CC) * P + local] = (int32_t)j;
        }
    }
    struct Run { uint32_t a, d, idesc; int first, len; };
    int64_t nt = 0, nr = 0, ns = 0, units16 = 0;
    std::vector<Run> step_runs;
    std::vector<int32_t> step_tiles;
    auto flush = [&](int ch, bool reuse, bool last) {
        const int ntile = (int)step_tiles.size(), nrun = (int)step_runs.size();
        if (fill) {
            step_off[ns] = (uint32_t)units16;
            const uint32_t meta = (uint32_t)ch | (reuse ? 0x40000000u : 0u) | (last ? 0x80000000u : 0u);
            step_meta[ns] = meta;
            uint32_t *hdr = reinterpret_cast<uint32_t *>(step_data + units16 * 16);
            hdr[0] = (uint32_t)ntile; hdr[1] = (uint32_t)nrun; hdr[2] = meta; hdr[3] = 0;
            uint32_t *rr = hdr + 4;
            for (int i = 0; i < nrun; ++i) {
                rr[4 * i + 0] = step_runs[i].a;
                rr[4 * i + 1] = (uint32_t)(step_runs[i].first * 32);   // B start offset, 16-byte units
                rr[4 * i + 2] = step_runs[i].d;
                rr[4 * i + 3] = step_runs[i].idesc;
            }
            uint8_t *td = reinterpret_cast<uint8_t *>(rr + 4 * nrun);
            for (int i = 0; i < ntile; ++i) memcpy(td + 64 * i, codes + (int64_t)step_tiles[i] * 64, 64);
        }
        units16 += 1 + nrun + 4 * (int64_t)ntile;
        nt += ntile; nr += nrun; ++ns;
        step_runs.clear(); step_tiles.clear();
    };
    // which cells hold at least one tile
    std::vector<uint8_t> cell_used((size_t)cells, 0);
    for (size_t i = 0; i < slot.size(); ++i)
        if (slot[i] >= 0) cell_used[i / ((size_t)CC * P)] = 1;
    for (int p = 0; p < NP; ++p) {
        uint32_t touched = 0;
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
                int l = 0;
                while (l < P) {
                    if (s[l] < 0) { ++l; continue; }
                    // a run must not mix rows already holding a partial sum with fresh rows:
                    // the first MMA into a row overwrites, later ones accumulate
                    const bool acc = (touched >> l) & 1u;
                    int e = l;
                    while (e < P && s[e] >= 0 && (((touched >> e) & 1u) != 0) == acc) ++e;
                    const int len = e - l;
                    if ((int)step_tiles.size() + len > MORTAR_STEP_TILES) {
                        flush(ch, !first_of_chunk, false);
                        first_of_chunk = false;
                    }
                    Run run;
                    run.a = (uint32_t)(cl * 2);                          // A start offset, 16-byte units
                    run.d = (uint32_t)(l * 16) | (acc ? 0x80000000u : 0u);
                    run.idesc = idesc_for(16 * len);
                    run.first = (int)step_tiles.size();
                    run.len = len;
                    step_runs.push_back(run);
                    for (int k = l; k < e; ++k) { step_tiles.push_back(s[k]); touched |= 1u << k; }
                    l = e;
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
    return build(row_ptr, col_idx, nullptr, R, C, swiglu, n_tiles, n_runs, n_steps, n_panels, data_units,
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
    return build(row_ptr, col_idx, codes, R, C, swiglu, &nt, &nr, &ns, &np, &du, step_data, step_off,
                 step_meta, panel_step_ptr, panel_mask);
}
