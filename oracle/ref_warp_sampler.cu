// Launch harness around the reference's OWN CUDA sampler kernel
// (`warp_sample_neighbors`).  Test infrastructure: the product never loads it.
//
// The two reference source files are included from where they lie in the
// reference checkout (the Makefile passes their paths), in the order the
// reference itself concatenates them before compiling
// (crates/aether-stream/src/gpu/kernels/sampler/mod.rs:22-27: common.cuh, then
// sampler.cu).  Nothing of them is copied into this repository; the built
// library goes to oracle/_ref/.  The launch shape follows
// sampler/mod.rs:199-207: 256 threads, one warp per requested node, grid
// clamped to [1, 65535] with the kernel striding past the cap.
#include <cuda_runtime.h>
#include <stdint.h>

#include REF_COMMON_CUH
#include REF_SAMPLER_CU

extern "C" int ref_warp_sample_launch(const unsigned long long *offsets_dev, const unsigned int *neighbors_dev,
                                      unsigned long long num_nodes, const unsigned long long *nodes_dev,
                                      unsigned int *output_dev, unsigned int *counts_dev, int node_count, int fanout,
                                      unsigned long long seed, unsigned int layer, void *stream) {
    if (node_count <= 0) return 0;
    const unsigned threads = 256;
    unsigned long long blocks = ((unsigned long long)node_count + threads / 32 - 1) / (threads / 32);
    if (blocks < 1) blocks = 1;
    if (blocks > 65535) blocks = 65535;
    warp_sample_neighbors<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
        offsets_dev, neighbors_dev, num_nodes, nodes_dev, output_dev, counts_dev, node_count, fanout, seed, layer);
    return (int)cudaGetLastError();
}
