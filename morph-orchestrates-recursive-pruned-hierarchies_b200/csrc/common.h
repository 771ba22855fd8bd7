// Shared declarations for the libmortar_b200 translation units.
#pragma once
#include <cstdint>
#include <cstdio>
#include "mortar_b200.h"

#define MORTAR_VERSION_STRING "mortar_b200 0.1 (sm_100a)"

// Geometry of the prefill panel schedule (shared by the host builder and the kernel).
#define MORTAR_PANEL_ROWS 16   // tile rows per panel = 256 fp32 accumulator columns of tensor memory
#define MORTAR_CHUNK_COLS 4    // tile columns per chunk = 64 features = one 128-byte swizzle row
#define MORTAR_STEP_SLOTS_I8 24 // slots (pairs of tiles) per step of the int8 schedule
#define MORTAR_STEP_TILES 48   // tile slots one B stage of the kernel holds (24 KB of bf16 tiles)

// Records the text of a failed CUDA runtime call for mortar_last_cuda_error().
void mortar_set_cuda_error(const char *what, const char *msg);

#define MORTAR_CUDA_CHECK(expr)                                         \
    do {                                                                \
        cudaError_t _e = (expr);                                        \
        if (_e != cudaSuccess) {                                        \
            mortar_set_cuda_error(#expr, cudaGetErrorString(_e));       \
            return MORTAR_ERR_CUDA;                                     \
        }                                                               \
    } while (0)

// Position of a tile element inside the 16-byte fragment word set of one lane.
//   lane = g*4 + t  (g = lane>>2, t = lane&3)
//   register i of the mma.m16n8k16 A fragment holds (row, col) / (row, col+1):
//     i=0: (g, 2t)   i=1: (g+8, 2t)   i=2: (g, 2t+8)   i=3: (g+8, 2t+8)
//   32-bit word w = slot>>1 of the lane's 16 bytes holds slots 2w and 2w+1; register
//   q = (slot&1)*4 + i keeps its low-column code in bits 2q..2q+1 and its high-column
//   code in bits 16+2q..16+2q+1.
static inline void mortar_frag_position(int row, int col, int *lane, int *reg, int *hi) {
    int g = row & 7, upper = row >> 3;
    int c8 = col & 7, right = col >> 3;
    *lane = g * 4 + (c8 >> 1);
    *reg = upper + 2 * right;
    *hi = c8 & 1;
}
