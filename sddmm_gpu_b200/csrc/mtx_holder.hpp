// A sparse matrix in host memory, 0-based row-sorted or unsorted COO: what
// sddmm_mtx_open and sddmm_gen_open hand to sddmm_mtx_read.
#pragma once
#include <cstdint>
#include <vector>

struct sddmm_mtx_s {
    int64_t M = 0, N = 0, nnz = 0;
    std::vector<int32_t> rows, cols;
    std::vector<float> vals;
};
