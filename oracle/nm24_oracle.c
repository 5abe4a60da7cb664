/*
 * CPU oracle, integer part: hard top-2-of-4 projection and its 2:4 metadata.
 * TEST INFRASTRUCTURE ONLY — never linked into or called by the product.
 *
 * Restates SparseLinear._hard_mask_from_soft, modes 'nm_2_4' and 'structured' (N:M = 2:4), of the
 * SparseForge reference (legacy/sparse_modeling.py:578-603, 720-735): per group of four along the
 * input dimension keep the two largest entries; columns beyond (cols/4)*4 stay 1. torch.topk's
 * tie order is unspecified; this path fixes it to "lower index wins", i.e. a stable descending
 * order, with NaN ordered as the largest value as torch does. The metadata nibble of a group is
 * i0 | (i1 << 2) (i0 < i1 the kept column offsets), two groups per byte, low nibble first.
 * Pinned against outputs of the reference (tests/golden/ties.npz) by tests/test_oracle_golden.py.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static int before(float a, int ia, float b, int ib) {
    /* does (a, ia) come before (b, ib) in the stable descending order? */
    int an = isnan(a), bn = isnan(b);
    if (an != bn) return an;         /* NaN first */
    if (!an && a != b) return a > b; /* larger first */
    return ia < ib;                  /* ties (and NaN vs NaN): lower index first */
}

void nm24_project(const float* soft, int64_t rows, int64_t cols, float* hard, uint8_t* meta) {
    const int64_t groups = cols / 4, bytes_per_row = (cols + 7) / 8;
    if (meta) memset(meta, 0, (size_t)(rows * bytes_per_row));
    for (int64_t r = 0; r < rows; ++r) {
        const float* s = soft + r * cols;
        for (int64_t g = 0; g < groups; ++g) {
            int rank[4] = {0, 0, 0, 0};
            for (int i = 0; i < 4; ++i)
                for (int j = 0; j < 4; ++j)
                    if (j != i && before(s[4 * g + j], j, s[4 * g + i], i)) rank[i]++;
            int i0 = -1, i1 = -1;
            for (int i = 0; i < 4; ++i) {
                const int keep = rank[i] < 2;
                if (hard) hard[r * cols + 4 * g + i] = keep ? 1.0f : 0.0f;
                if (keep) { if (i0 < 0) i0 = i; else i1 = i; }
            }
            if (meta) meta[r * bytes_per_row + g / 2] |= (uint8_t)((i0 | (i1 << 2)) << (4 * (g & 1)));
        }
        if (hard)
            for (int64_t c = groups * 4; c < cols; ++c) hard[r * cols + c] = 1.0f;
    }
}
