// Host-side helpers shared by the row-operator launchers: staged-tier geometry and grid sizing.
#pragma once

#include "ko_internal.h"
#include "../../include/ko_b200_tuning.h"

#include "../common/row_pipeline.h"

namespace ko {

constexpr int kStagedConsumerWarps = 16;
constexpr int kStagedThreads = (kStagedConsumerWarps + 1) * 32;

struct StagedPlan {
    RowPipeGeometry geo;
    int grid;
    size_t smem_bytes;
    bool ok;
};

// rows_per_group = rows one warp takes together; a stage holds a whole number of groups
inline StagedPlan plan_staged(long long rows, unsigned row_bytes, int rows_per_group, const ko_row_knobs_t &k,
                              const DeviceInfo &info) {
    StagedPlan p{};
    const int ctas = k.ctas_per_sm > 0 ? k.ctas_per_sm : 1;
    const size_t budget = (size_t)(info.max_smem_optin - 2048) / ctas - 1024;  // leave room for static smem
    int stage_rows = k.stage_rows;
    if (stage_rows <= 0) {
        // about 16 KB per bulk copy, at least one group
        const int groups = (int)((16384 + (size_t)rows_per_group * row_bytes - 1) / ((size_t)rows_per_group * row_bytes));
        stage_rows = rows_per_group * (groups > 0 ? groups : 1);
    }
    const size_t stage_bytes = (size_t)stage_rows * row_bytes;
    int stages = k.stages;
    if (stages <= 0) {
        const size_t target = ctas > 1 ? budget : (budget < (size_t)112 * 1024 ? budget : (size_t)112 * 1024);
        stages = (int)(target / stage_bytes);
        if (stages > 8) stages = 8;
    }
    p.geo.rows_per_stage = stage_rows;
    p.geo.stages = stages;
    p.geo.row_bytes = row_bytes;
    p.smem_bytes = row_pipe_smem_bytes(p.geo);
    p.ok = stages >= 2 && p.smem_bytes <= budget && stage_bytes < (1u << 20);
    long long grid = (long long)info.sm_count * ctas;
    const long long max_useful = (rows + stage_rows - 1) / stage_rows;
    if (grid > max_useful) grid = max_useful;
    p.grid = (int)(grid > 0 ? grid : 1);
    return p;
}

// raises a kernel's dynamic shared-memory limit once per (kernel, device) and only when it grows
int ensure_dynamic_smem(const void *kernel, size_t bytes);

// Launch `kernel` with thread-block clusters of `cluster` blocks along x (grid must be a multiple of it).
template <typename... KernelArgs, typename... Args>
int launch_clustered_smem(void (*kernel)(KernelArgs...), unsigned grid, unsigned block, unsigned cluster, size_t smem,
                          cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    KO_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...));
    return KO_OK;
}

// Launch `kernel` so that its blocks may be scheduled while the stream's previous kernel drains
// (programmatic dependent launch); the kernel orders itself with ko::grid_dependency_wait().
template <typename... KernelArgs, typename... Args>
int launch_overlapped(void (*kernel)(KernelArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    KO_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...));
    return KO_OK;
}

// Both of the above: clusters of `cluster` blocks along x, launched with programmatic stream serialization.
template <typename... KernelArgs, typename... Args>
int launch_clustered_overlapped(void (*kernel)(KernelArgs...), unsigned grid, unsigned block, unsigned cluster, size_t smem,
                                cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    KO_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...));
    return KO_OK;
}

// how many clusters of `cluster` blocks of `kernel` the current device can hold at once (at least 1)
inline int max_resident_clusters(const void *kernel, unsigned block, unsigned cluster, size_t smem, int *out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    KO_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    *out = n > 0 ? n : 1;
    return KO_OK;
}

template <typename... KernelArgs, typename... Args>
int launch_clustered(void (*kernel)(KernelArgs...), unsigned grid, unsigned block, unsigned cluster, cudaStream_t s,
                     Args... args) {
    return launch_clustered_smem(kernel, grid, block, cluster, 0, s, args...);
}

// cluster size (power of two, <= 8) so that a block's slice of `nvec` vectors fits `per_block` vectors;
// 0 when even 8 blocks are not enough
inline int cluster_size_for(int nvec, int per_block, int wanted) {
    int c = wanted > 0 ? wanted : 2;
    while (c < 8 && (nvec + c - 1) / c > per_block) c *= 2;
    return (nvec + c - 1) / c <= per_block ? c : 0;
}

inline unsigned clamp_grid(long long wanted, long long cap) {
    if (cap > 0 && wanted > cap) wanted = cap;
    if (wanted > 0x7fffffffLL) wanted = 0x7fffffffLL;
    return (unsigned)(wanted > 0 ? wanted : 1);
}

}  // namespace ko
