// Internal declarations shared by the translation units of libaethergpu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "../../include/aethergpu.h"

struct ag_graph {
    int device = 0;
    uint64_t num_nodes = 0, num_edges = 0;
    uint64_t *offsets = nullptr;  // device, num_nodes + 1
    uint32_t *dst = nullptr;      // device, num_edges
    float *weights = nullptr;     // device, num_edges or null
};

struct ag_features {
    int device = 0;
    uint64_t num_nodes = 0;   // rows of the whole store
    uint64_t row_begin = 0;   // first row held here (vertex-range shard)
    uint64_t rows = 0;        // rows held here
    uint64_t dim = 0;
    int dtype = AG_F32;
    uint8_t *payload = nullptr;  // device, rows * dim * elem_size
    uint32_t *err = nullptr;     // device, sticky error bits
    bool owns_payload = true;
};

namespace ag {

inline uint32_t elem_size(int dtype) { return dtype == AG_F32 ? 4u : 2u; }

struct GatherArgs {
    const uint8_t *payload;
    uint64_t row_begin, rows;
    uint32_t row_bytes, dim;
    const void *ids;
    int ids64;
    uint64_t n;
    const uint32_t *n_dev;
    float *out;
    uint32_t *err;
};

cudaError_t launch_gather(const GatherArgs &a, int dtype, cudaStream_t st);
cudaError_t launch_gather_group(const GatherArgs *group_dev, uint32_t n_batches, uint32_t row_bytes,
                                uint32_t dim, uint64_t n_bound, bool aligned, int dtype, cudaStream_t st);
cudaError_t launch_encode(const float *src, void *dst, uint64_t count, int dtype, cudaStream_t st);
int gather_grid_blocks(uint64_t n, uint32_t row_bytes);

// Device-side validation of a CSR: offsets monotone, offsets[n] == e, dst < n.
// Writes a non-zero code to *flag_dev on failure.
cudaError_t launch_validate_csr(const uint64_t *offsets, const uint32_t *dst, uint64_t n,
                                uint64_t e, uint64_t dst_bound, uint32_t *flag_dev,
                                cudaStream_t st);
cudaError_t launch_degrees(const uint64_t *offsets, uint64_t num_nodes, const uint32_t *ids,
                           uint64_t n, uint32_t *out, cudaStream_t st);

// Sorts n keys (row << 32 | value) and builds the CSR over num_rows rows from them
// (rows ascending, values ascending within a row).  Consumes (frees) keys.
int32_t keys_to_sorted_csr(uint64_t *keys, uint64_t n, uint64_t num_rows, uint64_t **offsets_out,
                           uint32_t **vals_out);

}  // namespace ag
