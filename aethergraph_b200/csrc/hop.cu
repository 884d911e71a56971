// One-hop Philox reservoir sampling: the fast-mode sampler of the reference
// (CPU: crates/aethergraph-core/src/internal/philox.rs:59-82 `reservoir_sample`;
// GPU: crates/aether-stream/src/gpu/kernels/sampler/sampler.cu `warp_sample_neighbors`,
// launched by sampler/mod.rs:180-230).  Same inputs, same outputs, same bits:
// for every requested node a row of `fanout` slots —
//   degree == 0 or node outside the graph: count 0;
//   fanout > 32: `fanout` draws with replacement, slot d = row[philox(d) % degree];
//   fanout >= degree: the row itself, count = degree;
//   else Algorithm R keyed by the scan position t (draw t decides j = r % (t + 1)),
// unused slots hold AG_SAMPLE_PAD, counts[row] says how many are real.
//
// Algorithm R looks sequential in t, but every decision j(t) is a pure function
// of (seed, layer, node, t), and the reservoir's final slot j simply holds the
// element with the LARGEST t that chose j (or element j itself if none did).  So
// the lanes of a warp evaluate the t's in parallel and keep a per-slot maximum;
// no lane waits for another and the result is bit-identical.
#include "common.cuh"
#include "internal.h"

namespace ag {
namespace {

constexpr int kHopThreads = 256;

__global__ void __launch_bounds__(kHopThreads)
k_hop_reservoir(const uint64_t *__restrict__ offsets, const uint32_t *__restrict__ neighbors, uint64_t num_nodes,
                uint64_t num_edges, const uint64_t *__restrict__ nodes, uint32_t *__restrict__ output,
                uint32_t *__restrict__ counts, uint64_t node_count, uint32_t fanout, uint64_t seed, uint32_t layer) {
    __shared__ unsigned long long s_last[kHopThreads / 32][32];  // per warp: largest t that chose slot j
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t first = ((uint64_t)blockIdx.x * kHopThreads + threadIdx.x) >> 5;
    const uint64_t stride = ((uint64_t)gridDim.x * kHopThreads) >> 5;
    for (uint64_t row = first; row < node_count; row += stride) {
        uint32_t *out = output + row * fanout;
        const uint64_t node = nodes[row];
        uint64_t begin = 0, degree = 0;
        if (node < num_nodes) {
            begin = __ldg(offsets + node);
            const uint64_t end = __ldg(offsets + node + 1);
            degree = (end >= begin && end <= num_edges) ? end - begin : 0;
        }
        uint32_t taken = 0;
        if (degree == 0) {
            taken = 0;
        } else if (fanout > 32) {
            for (uint32_t d = lane; d < fanout; d += 32) {
                const uint32_t r = philox_u32(seed, layer, node, d);
                out[d] = ld_stream_u32(neighbors + begin + (r % degree));
            }
            taken = fanout;
        } else if ((uint64_t)fanout >= degree) {
            for (uint64_t i = lane; i < degree; i += 32) out[i] = ld_stream_u32(neighbors + begin + i);
            taken = (uint32_t)degree;
        } else {
            s_last[warp][lane] = (unsigned long long)lane;  // slot j starts with element j
            __syncwarp();
            for (uint64_t t = (uint64_t)fanout + lane; t < degree; t += 32) {
                const uint32_t r = philox_u32(seed, layer, node, (uint32_t)t);
                const uint32_t j = r % (uint32_t)(t + 1);
                if (j < fanout) atomicMax(&s_last[warp][j], (unsigned long long)t);
            }
            __syncwarp();
            if ((uint32_t)lane < fanout) out[lane] = ld_stream_u32(neighbors + begin + s_last[warp][lane]);
            taken = fanout;
            __syncwarp();
        }
        for (uint32_t i = taken + lane; i < fanout; i += 32) out[i] = AG_SAMPLE_PAD;
        if (lane == 0) counts[row] = taken;
    }
}

}  // namespace
}  // namespace ag

using namespace ag;

extern "C" int32_t ag_sample_hop_reservoir(const ag_graph *g, const uint64_t *nodes_dev, uint64_t node_count,
                                           uint32_t fanout, uint64_t seed, uint32_t layer,
                                           uint32_t *neighbors_out_dev, uint32_t *counts_out_dev, void *stream) {
    if (!g || !neighbors_out_dev || !counts_out_dev || (!nodes_dev && node_count))
        return fail(AG_ERR_VALUE, "ag_sample_hop_reservoir: null argument");
    if (fanout == 0) return fail(AG_ERR_VALUE, "fanout must be >= 1");
    if (node_count == 0) return AG_OK;
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const uint64_t blocks = std::min<uint64_t>((node_count + kHopThreads / 32 - 1) / (kHopThreads / 32), (uint64_t)kSMs * 32);
    k_hop_reservoir<<<(uint32_t)std::max<uint64_t>(blocks, 1), kHopThreads, 0, (cudaStream_t)stream>>>(
        g->offsets, g->dst, g->num_nodes, g->num_edges, nodes_dev, neighbors_out_dev, counts_out_dev, node_count, fanout,
        seed, layer);
    AG_CUDA(cudaGetLastError());
    return AG_OK;
}
