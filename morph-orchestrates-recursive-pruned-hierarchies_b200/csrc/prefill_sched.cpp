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
// boundaries); empty cells produce no step.  step_chunk[i] = chunk index, with bit 30 set
// when the step reuses the activation chunk of the previous step and bit 31 set when it is
// the last step on that chunk.
static int build(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes, int32_t R,
                 int32_t C, int32_t swiglu, int64_t *n_tiles_out, int64_t *n_runs_out,
                 int64_t *n_steps_out, int32_t *n_panels_out, uint8_t *tiles, uint32_t *runs,
                 int32_t *panel_step_ptr, int32_t *step_tile_ptr, int32_t *step_run_ptr,
                 uint32_t *step_chunk, uint32_t *panel_mask) {
    if (!row_ptr || !n_tiles_out || !n_runs_out || !n_steps_out || !n_panels_out) return MORTAR_ERR_NULL;
    if (R <= 0 || C <= 0 || C > 65534) return MORTAR_ERR_SHAPE;
    if (swiglu && (R % 2)) return MORTAR_ERR_SHAPE;
    const int units = swiglu ? R / 2 : R;
    const int per_panel = swiglu ? P / 2 : P;
    const int NP = (units + per_panel - 1) / per_panel;
    const int NC = (C + CC - 1) / CC;
    const bool fill = tiles != nullptr;
    if (fill && (!runs || !panel_step_ptr || !step_tile_ptr || !step_run_ptr || !step_chunk ||
                 !panel_mask || !col_idx || !codes))
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
    int64_t nt = 0, nr = 0, ns = 0;
    for (int p = 0; p < NP; ++p) {
        uint32_t touched = 0;
        if (fill) panel_step_ptr[p] = (int32_t)ns;
        for (int ch = 0; ch < NC; ++ch) {
            const size_t cell = (size_t)p * NC + ch;
            int in_step = 0;            // tiles already placed in the open step
            bool step_open = false, first_of_chunk = true;
            int64_t last_step = -1;
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
                    if (!step_open || in_step + len > MORTAR_STEP_TILES) {
                        if (fill) {
                            step_tile_ptr[ns] = (int32_t)nt;
                            step_run_ptr[ns] = (int32_t)nr;
                            step_chunk[ns] = (uint32_t)ch | (first_of_chunk ? 0u : 0x40000000u);
                        }
                        last_step = ns;
                        ++ns;
                        step_open = true; first_of_chunk = false; in_step = 0;
                    }
                    if (fill) {
                        uint32_t *rr = runs + nr * 4;
                        rr[0] = (uint32_t)(cl * 2);                 // A start offset, 16-byte units
                        rr[1] = (uint32_t)(in_step * 32);           // B start offset, 16-byte units
                        rr[2] = (uint32_t)(l * 16) | (acc ? 0x80000000u : 0u);
                        rr[3] = idesc_for(16 * len);
                        for (int k = l; k < e; ++k)
                            memcpy(tiles + (nt + (k - l)) * 64, codes + (int64_t)s[k] * 64, 64);
                    }
                    for (int k = l; k < e; ++k) touched |= 1u << k;
                    nt += len; nr += 1; in_step += len;
                    l = e;
                }
            }
            if (fill && last_step >= 0) step_chunk[last_step] |= 0x80000000u;
        }
        if (fill) panel_mask[p] = touched;
    }
    if (nt > INT32_MAX || nr > INT32_MAX || ns > INT32_MAX) return MORTAR_ERR_CAPACITY;
    if (fill) {
        panel_step_ptr[NP] = (int32_t)ns;
        step_tile_ptr[ns] = (int32_t)nt;
        step_run_ptr[ns] = (int32_t)nr;
    }
    *n_tiles_out = nt; *n_runs_out = nr; *n_steps_out = ns; *n_panels_out = NP;
    return MORTAR_OK;
}

extern "C" int mortar_sched_sizes(const int32_t *row_ptr, const uint16_t *col_idx, int32_t R, int32_t C,
                                  int32_t swiglu, int64_t *n_tiles, int64_t *n_runs, int64_t *n_steps,
                                  int32_t *n_panels) {
    return build(row_ptr, col_idx, nullptr, R, C, swiglu, n_tiles, n_runs, n_steps, n_panels, nullptr,
                 nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
}

extern "C" int mortar_build_sched(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes,
                                  int32_t R, int32_t C, int64_t nnz, int32_t swiglu, uint8_t *tiles,
                                  uint32_t *runs, int32_t *panel_step_ptr, int32_t *step_tile_ptr,
                                  int32_t *step_run_ptr, uint32_t *step_chunk, uint32_t *panel_mask) {
    int v = mortar_validate_bcsr(row_ptr, col_idx, codes, R, C, nnz);
    if (v != MORTAR_OK) return v;
    if (!tiles) return MORTAR_ERR_NULL;
    int64_t nt, nr, ns; int32_t np;
    return build(row_ptr, col_idx, codes, R, C, swiglu, &nt, &nr, &ns, &np, tiles, runs, panel_step_ptr,
                 step_tile_ptr, step_run_ptr, step_chunk, panel_mask);
}
