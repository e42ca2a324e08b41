// Launch shapes per problem shape: the table the library consults before it falls back on its
// built-in rules.  Role of the reference's tuned-parameter tables and their lookup
// (scripts/optima.csv, scripts/optima-fixed-max_slowdown.csv:44-49, `config_algorithm` in
// scripts/config.sh:98-214, which pick block size / batch size / register tiling per (q, k, dim)
// for its kernels); here the lookup is inside the library, so every caller gets the tuned shape.
//
// The rows live in tuning_table.inc, which bits-knn-jpdc2024_b200/tune.py regenerates from a sweep
// on the GPU at hand.  A row applies to the first key it matches, rows are ordered by key.
#pragma once

#include <cstdint>

namespace bitsknn
{

// `bits` selection: key = (k <= k_max, row slices per launch <= rows_max).
struct select_shape
{
    int k_max;
    int64_t rows_max;
    int threads;     // block size: 256, 512 or 1024
    int ipt;         // list pairs per thread; threads * ipt >= k_max
    int stage_bytes; // bytes per stage of the row stream
    int stages;
    int merge_pct;   // fold the buffer at this percentage of a list's length
    int unroll;      // 128-bit vectors per thread under one warp vote (2 or 4)
    int blocks_wanted; // row slices the automatic split aims at on a 148-SM device (0: rule of thumb)
};

// FP32 fused search: key = (dim <= dim_max, k <= k_max); which kernel runs when a workspace is given.
struct fused_shape
{
    int dim_max;
    int k_max;
    int tiled; // 1: 128 x 128 tiled kernel, 0: 8-queries-per-block kernel
};

inline constexpr select_shape SELECT_SHAPES[] = {
#define BITSKNN_SELECT_ROW(...) {__VA_ARGS__},
#define BITSKNN_FUSED_ROW(...)
#include "tuning_table.inc"
#undef BITSKNN_SELECT_ROW
#undef BITSKNN_FUSED_ROW
};

inline constexpr fused_shape FUSED_SHAPES[] = {
#define BITSKNN_SELECT_ROW(...)
#define BITSKNN_FUSED_ROW(...) {__VA_ARGS__},
#include "tuning_table.inc"
#undef BITSKNN_SELECT_ROW
#undef BITSKNN_FUSED_ROW
};

inline const select_shape* find_select_shape(int k, int64_t rows)
{
    for (const auto& row : SELECT_SHAPES)
    {
        if (k <= row.k_max && rows <= row.rows_max && row.threads * row.ipt >= k)
        {
            return &row;
        }
    }
    return nullptr;
}

inline const fused_shape* find_fused_shape(int dim, int k)
{
    for (const auto& row : FUSED_SHAPES)
    {
        if (dim <= row.dim_max && k <= row.k_max)
        {
            return &row;
        }
    }
    return nullptr;
}

} // namespace bitsknn
