// Host-side format work: validation of the canonical tile-16 BCSR, construction of the
// 8-tile-group stream layout the kernels read, its inverse, and the splitter that turns
// the reference's larger square blocks into 16x16 tiles.  No GPU calls in this file.
#include <cstring>
#include <vector>
#include "common.h"

static thread_local char g_cuda_err[512] = "";

void mortar_set_cuda_error(const char *what, const char *msg) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, msg);
}

extern "C" const char *mortar_last_cuda_error(void) { return g_cuda_err; }
extern "C" const char *mortar_version(void) { return MORTAR_VERSION_STRING; }

extern "C" const char *mortar_status_string(int s) {
    switch (s) {
        case MORTAR_OK: return "ok";
        case MORTAR_ERR_NULL: return "required pointer is NULL";
        case MORTAR_ERR_SHAPE: return "bad shape: zero, negative or not a multiple of 16";
        case MORTAR_ERR_ROWPTR: return "row pointer not monotone or wrong end value";
        case MORTAR_ERR_COLIDX: return "column index out of range or not ascending inside a row";
        case MORTAR_ERR_CODE: return "a 2-bit code field holds the unused value 3";
        case MORTAR_ERR_ALIGN: return "pointer or stride not aligned as documented";
        case MORTAR_ERR_DTYPE: return "unknown dtype, mode or plane count";
        case MORTAR_ERR_CAPACITY: return "buffer or built-in limit too small";
        case MORTAR_ERR_CUDA: return "CUDA runtime error";
        case MORTAR_ERR_UNSUPPORTED: return "unsupported combination";
        default: return "unknown status";
    }
}

extern "C" int mortar_validate_bcsr(const int32_t *row_ptr, const uint16_t *col_idx,
                                    const uint8_t *codes, int32_t R, int32_t C, int64_t nnz) {
    if (!row_ptr || (nnz > 0 && (!col_idx || !codes))) return MORTAR_ERR_NULL;
    if (R <= 0 || C <= 0 || C > 65534 || nnz < 0) return MORTAR_ERR_SHAPE;
    if (row_ptr[0] != 0 || row_ptr[R] != nnz) return MORTAR_ERR_ROWPTR;
    for (int r = 0; r < R; ++r) {
        if (row_ptr[r + 1] < row_ptr[r]) return MORTAR_ERR_ROWPTR;
        if (row_ptr[r + 1] > nnz) return MORTAR_ERR_ROWPTR;
        for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
            if (col_idx[j] >= C) return MORTAR_ERR_COLIDX;
            if (j > row_ptr[r] && col_idx[j] <= col_idx[j - 1]) return MORTAR_ERR_COLIDX;
        }
    }
    for (int64_t i = 0; i < nnz * 64; ++i) {
        uint8_t b = codes[i];
        // a field equals 3 iff both of its bits are set
        if (b & (b >> 1) & 0x55) return MORTAR_ERR_CODE;
    }
    return MORTAR_OK;
}

extern "C" int64_t mortar_stream_groups(const int32_t *row_ptr, int32_t R) {
    if (!row_ptr) return MORTAR_ERR_NULL;
    if (R <= 0) return MORTAR_ERR_SHAPE;
    int64_t g = 0;
    for (int r = 0; r < R; ++r) {
        int64_t n = (int64_t)row_ptr[r + 1] - row_ptr[r];
        if (n < 0) return MORTAR_ERR_ROWPTR;
        g += (n + 7) / 8;
    }
    return g;
}

static inline int tile_code(const uint8_t *tile, int row, int col) {   // stored value 0..2
    return (tile[row * 4 + (col >> 2)] >> (2 * (col & 3))) & 3;
}

extern "C" int mortar_build_stream(const int32_t *row_ptr, const uint16_t *col_idx,
                                   const uint8_t *codes, int32_t R, int32_t C, int64_t nnz,
                                   int32_t *grp_ptr, uint16_t *grp_cols, uint8_t *grp_codes) {
    int v = mortar_validate_bcsr(row_ptr, col_idx, codes, R, C, nnz);
    if (v != MORTAR_OK) return v;
    if (!grp_ptr || !grp_cols || !grp_codes) return MORTAR_ERR_NULL;
    int64_t g = 0;
    grp_ptr[0] = 0;
    for (int r = 0; r < R; ++r) {
        int64_t lo = row_ptr[r], hi = row_ptr[r + 1];
        for (int64_t j0 = lo; j0 < hi; j0 += 8, ++g) {
            uint32_t *words = reinterpret_cast<uint32_t *>(grp_codes + g * 512);
            // every field starts as stored value 1 (code 0)
            for (int i = 0; i < 128; ++i) words[i] = 0x55555555u;
            for (int s = 0; s < 8; ++s) {
                int64_t j = j0 + s;
                if (j >= hi) {   // padding slot: marked by the column sentinel, never read
                    grp_cols[g * 8 + s] = 0xFFFFu;
                    continue;
                }
                grp_cols[g * 8 + s] = col_idx[j];
                const uint8_t *tile = codes + j * 64;
                for (int row = 0; row < 16; ++row)
                    for (int col = 0; col < 16; ++col) {
                        int lane, reg, hi16;
                        mortar_frag_position(row, col, &lane, &reg, &hi16);
                        int q = (s & 1) * 4 + reg;
                        int bit = 2 * q + 16 * hi16;
                        uint32_t &w = words[lane * 4 + (s >> 1)];
                        w = (w & ~(3u << bit)) | ((uint32_t)tile_code(tile, row, col) << bit);
                    }
            }
        }
        if (g > INT32_MAX) return MORTAR_ERR_CAPACITY;
        grp_ptr[r + 1] = (int32_t)g;
    }
    return MORTAR_OK;
}

extern "C" int mortar_unpack_stream(const int32_t *grp_ptr, const uint16_t *grp_cols,
                                    const uint8_t *grp_codes, const int32_t *row_ptr, int32_t R,
                                    uint16_t *col_idx, uint8_t *codes) {
    if (!grp_ptr || !grp_cols || !grp_codes || !row_ptr || !col_idx || !codes) return MORTAR_ERR_NULL;
    if (R <= 0) return MORTAR_ERR_SHAPE;
    for (int r = 0; r < R; ++r) {
        int64_t lo = row_ptr[r], hi = row_ptr[r + 1];
        int64_t g = grp_ptr[r];
        for (int64_t j0 = lo; j0 < hi; j0 += 8, ++g) {
            const uint32_t *words = reinterpret_cast<const uint32_t *>(grp_codes + g * 512);
            for (int s = 0; s < 8 && j0 + s < hi; ++s) {
                int64_t j = j0 + s;
                col_idx[j] = grp_cols[g * 8 + s];
                uint8_t *tile = codes + j * 64;
                memset(tile, 0, 64);
                for (int row = 0; row < 16; ++row)
                    for (int col = 0; col < 16; ++col) {
                        int lane, reg, hi16;
                        mortar_frag_position(row, col, &lane, &reg, &hi16);
                        int q = (s & 1) * 4 + reg;
                        int bit = 2 * q + 16 * hi16;
                        uint32_t st = (words[lane * 4 + (s >> 1)] >> bit) & 3u;
                        tile[row * 4 + (col >> 2)] |= (uint8_t)(st << (2 * (col & 3)));
                    }
            }
        }
        if (g != grp_ptr[r + 1]) return MORTAR_ERR_ROWPTR;
    }
    return MORTAR_OK;
}

extern "C" int mortar_split_blocks(const int32_t *offsets, const int16_t *column_indices,
                                   const uint8_t *packed, int32_t Rb, int32_t Cb, int32_t blocking,
                                   int32_t drop_zero, int32_t *row_ptr_out, uint16_t *col_idx_out,
                                   uint8_t *codes_out, int64_t *nnz_out) {
    if (!offsets || !column_indices || !packed || !row_ptr_out || !nnz_out) return MORTAR_ERR_NULL;
    if (Rb <= 0 || Cb <= 0 || blocking < 16 || blocking % 16) return MORTAR_ERR_SHAPE;
    const int tpb = blocking / 16;
    if ((int64_t)Cb * tpb > 65534) return MORTAR_ERR_SHAPE;
    if (offsets[0] != 0) return MORTAR_ERR_ROWPTR;
    const int64_t bytes_per_row = blocking / 4;           // one block row of codes
    const int64_t bytes_per_block = (int64_t)blocking * bytes_per_row;
    int64_t nnz = 0;
    row_ptr_out[0] = 0;
    std::vector<uint8_t> tile(64);
    for (int rb = 0; rb < Rb; ++rb) {
        if (offsets[rb + 1] < offsets[rb]) return MORTAR_ERR_ROWPTR;
        for (int tr = 0; tr < tpb; ++tr) {
            for (int64_t j = offsets[rb]; j < offsets[rb + 1]; ++j) {
                int cb = column_indices[j];
                if (cb < 0 || cb >= Cb) return MORTAR_ERR_COLIDX;
                if (j > offsets[rb] && column_indices[j] <= column_indices[j - 1]) return MORTAR_ERR_COLIDX;
                const uint8_t *blk = packed + j * bytes_per_block;
                for (int tc = 0; tc < tpb; ++tc) {
                    bool any = false;
                    for (int row = 0; row < 16; ++row) {
                        const uint8_t *src = blk + (int64_t)(tr * 16 + row) * bytes_per_row + tc * 4;
                        for (int b = 0; b < 4; ++b) {
                            uint8_t v = src[b];
                            if (v & (v >> 1) & 0x55) return MORTAR_ERR_CODE;
                            tile[row * 4 + b] = v;
                            any |= (v != 0x55);
                        }
                    }
                    if (drop_zero && !any) continue;
                    if (codes_out) {
                        if (!col_idx_out) return MORTAR_ERR_NULL;
                        col_idx_out[nnz] = (uint16_t)(cb * tpb + tc);
                        memcpy(codes_out + nnz * 64, tile.data(), 64);
                    }
                    ++nnz;
                }
            }
            if (nnz > INT32_MAX) return MORTAR_ERR_CAPACITY;
            row_ptr_out[rb * tpb + tr + 1] = (int32_t)nnz;
        }
    }
    *nnz_out = nnz;
    return MORTAR_OK;
}
