// Grouping: stable token -> expert grouping on the GPU (upstream src/grouping.rs:12-111 and the six kernels
// of native/grouping.cu).  Same result contract:
//   ids[u]      distinct expert ids of the window, ascending
//   count[0]    their number
//   members[u]  row * 32 + slot of every row that picked ids[u], ascending rows, then -1 up to maxm;
//               rows u >= count are all -1
// One launch for any window size (upstream: one block for <= 32 rows, five launches up to 8192 rows): CTA e
// owns expert e.  It first builds the bitmap of used experts from the picks itself (so it knows its place
// among the used experts without a second kernel or a global scan), then walks the rows in order, 1024 at a
// time, and compacts the rows that picked e with a block scan.  Nothing is ordered by atomics: the shared-
// memory atomicOr only sets bits.  A row that names an expert twice counts once, with its first slot, as in
// upstream's row-bitmap.
#include <algorithm>
#include <new>

#include "common.cuh"

namespace gf {
int check_config(const glmflash_config *cfg, size_t cfg_bytes, int max_rows_limit);

constexpr int GROUP_THREADS = 1024;

__global__ void __launch_bounds__(GROUP_THREADS) grouping_kernel(const int *__restrict__ picks, int rows, int slots, int E1,
                                                                int maxm, int *__restrict__ ids, int *__restrict__ count,
                                                                int *__restrict__ members) {
    __shared__ uint32_t used[32];                 // E1 <= 1024
    __shared__ int warp_sums[32];
    __shared__ int base_sh;
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();                                   // picks may be the previous kernel's output; ids / members its input
    pdl_launch_dependents();
    if (tid < 32) used[tid] = 0u;
    if (tid == 0) base_sh = 0;
    __syncthreads();
    const int total = rows * slots;
    for (int i = tid; i < total; i += GROUP_THREADS) {
        const int p = picks[i];
        if (p >= 0 && p < E1) atomicOr(&used[p >> 5], 1u << (p & 31));
    }
    __syncthreads();
    int place = 0, n_used = 0;
    for (int wd = 0; wd < 32; ++wd) {
        const uint32_t b = used[wd];
        n_used += __popc(b);
        if (wd < (e >> 5)) place += __popc(b);
        else if (wd == (e >> 5)) place += __popc(b & ((1u << (e & 31)) - 1u));
    }
    const bool mine = (used[e >> 5] >> (e & 31)) & 1u;
    if (e == 0 && tid == 0) *count = n_used;
    if (mine && tid == 0) ids[place] = e;
    if (!mine && e >= n_used && tid == 0) ids[e] = -1;       // tail of ids: not read by consumers, kept tidy

    if (mine) {
        int *out = members + (size_t)place * maxm;
        for (int r0 = 0; r0 < rows; r0 += GROUP_THREADS) {
            const int r = r0 + tid;
            int slot = -1;
            if (r < rows)
                for (int s = slots - 1; s >= 0; --s)
                    if (picks[r * slots + s] == e) slot = s;     // first matching slot wins
            const int flag = slot >= 0;
            // block exclusive scan of flag
            const uint32_t ball = __ballot_sync(0xffffffffu, flag);
            const int in_warp = __popc(ball & ((1u << lane) - 1u));
            if (lane == 0) warp_sums[warp] = __popc(ball);
            __syncthreads();
            int before = 0, chunk = 0;
            for (int w2 = 0; w2 < GROUP_THREADS / 32; ++w2) {
                const int v = warp_sums[w2];
                if (w2 < warp) before += v;
                chunk += v;
            }
            const int base = base_sh;
            if (flag) {
                const int off = base + before + in_warp;
                if (off < maxm) out[off] = r * 32 + slot;
            }
            __syncthreads();
            if (tid == 0) base_sh = base + chunk;
            __syncthreads();
        }
        for (int j = min(base_sh, maxm) + tid; j < maxm; j += GROUP_THREADS) out[j] = -1;
    }
    // rows of `members` beyond the used ones: row e is unused exactly when e >= n_used
    if (e >= n_used)
        for (int j = tid; j < maxm; j += GROUP_THREADS) members[(size_t)e * maxm + j] = -1;
}

int launch_grouping(cudaStream_t s, const int *picks, int rows, int slots, int E1, int maxm, int *ids, int *count,
                    int *members, bool pdl) {
    return launch_k(grouping_kernel, dim3(E1), dim3(GROUP_THREADS), 0, s, pdl, picks, rows, slots, E1, maxm, ids, count,
                    members);
}
}  // namespace gf

using namespace gf;

struct glmflash_grouping {
    glmflash_config cfg;
    int *ids = nullptr, *count = nullptr, *members = nullptr;
};

extern "C" int glmflash_grouping_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_grouping **out) {
    GF_REQUIRE(out != nullptr, "out is null");
    *out = nullptr;
    if (check_config(cfg, cfg_bytes, 8192)) return -1;       // upstream: 1..=8192, src/grouping.rs:30
    glmflash_grouping *g = new (std::nothrow) glmflash_grouping();
    GF_REQUIRE(g != nullptr, "out of host memory");
    g->cfg = *cfg;
    const size_t E1 = cfg->experts + 1;
    cudaError_t e1 = cudaMalloc((void **)&g->ids, E1 * 4), e2 = cudaMalloc((void **)&g->count, 4),
                e3 = cudaMalloc((void **)&g->members, E1 * cfg->max_rows * 4);
    if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess) {
        glmflash_grouping_free(g);
        return fail_cuda(e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3), "cudaMalloc(grouping)");
    }
    cudaMemset(g->ids, 0xff, E1 * 4);
    cudaMemset(g->count, 0, 4);
    cudaMemset(g->members, 0xff, E1 * cfg->max_rows * 4);
    *out = g;
    return 0;
}

extern "C" void glmflash_grouping_free(glmflash_grouping *g) {
    if (!g) return;
    cudaFree(g->ids); cudaFree(g->count); cudaFree(g->members);
    delete g;
}

extern "C" int glmflash_grouping_run(glmflash_grouping *g, void *stream, const int32_t *picks, int rows) {
    GF_REQUIRE(g && picks, "null argument");
    GF_REQUIRE(rows > 0 && rows <= g->cfg.max_rows, "grouping rows exceed scratch");
    return launch_grouping((cudaStream_t)stream, picks, rows, g->cfg.slots, g->cfg.experts + 1, g->cfg.max_rows, g->ids,
                           g->count, g->members, g->cfg.pdl != 0);
}

extern "C" const int32_t *glmflash_grouping_ids(const glmflash_grouping *g) { return g ? g->ids : nullptr; }
extern "C" const int32_t *glmflash_grouping_count(const glmflash_grouping *g) { return g ? g->count : nullptr; }
extern "C" const int32_t *glmflash_grouping_members(const glmflash_grouping *g) { return g ? g->members : nullptr; }
