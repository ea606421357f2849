// Static persistent tile schedule shared by the GEMM kernels.
//
// Tiles = row blocks (128 rows of sorted_token_ids, one expert each) x column tiles. CTA b walks tiles
// b, b + gridDim.x, ...  Tile ids are laid out in groups of kGroupM consecutive row blocks x all column
// tiles, row block fastest, so the CTAs running at the same time share weight tiles through L2.
#pragma once
#include <stdint.h>

namespace pmoe {

constexpr int kBlockM = 128;
constexpr int kGroupM = 8;

struct Coord {
    int m_blk, n_tile;
};

__device__ __forceinline__ Coord tile_coord(int t, int m_blocks, int n_tiles) {
    const int per_group = kGroupM * n_tiles;
    const int g = t / per_group;
    const int first = g * kGroupM;
    const int gsz = min(kGroupM, m_blocks - first);
    const int local = t - g * per_group;
    Coord c;
    c.m_blk = first + local % gsz;
    c.n_tile = local / gsz;
    return c;
}

// number of live 128-row blocks: num_tokens_post_padded clamped to the allocated length
__device__ __forceinline__ int live_row_blocks(const int32_t *npp_ptr, int sorted_num) {
    int npp = *npp_ptr;
    npp = max(0, min(npp, sorted_num));
    return npp / kBlockM;
}

}  // namespace pmoe
