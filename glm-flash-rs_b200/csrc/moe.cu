// Moe: grouping -> experts -> combine for one window (upstream src/moe.rs:11-182 for one row,
// src/model_verifier.rs:1291-1305 and src/batch.rs:1160-1210 for windows and chunks), plus the rank-ordered
// sum that follows the cross-GPU all-gather (upstream src/model.rs:485-496).
#include <algorithm>
#include <new>

#include <stdlib.h>

#include "common.cuh"
#include "owners.cuh"

namespace gf {
int experts_run_fused(glmflash_experts *e, cudaStream_t s, const glmflash_weights *w, const void *input, int x_stride,
                      const int32_t *picks, int rows);

// out[r][d] = sum_{s < slots-1, expert computed here} w[r][s] * Y[r*slots+s][d]  (+ Y[shared pair] if computed here)
// fp32, ascending slot order, shared last: the order of the oracle's combine.
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ Y, const int *__restrict__ picks,
                                                      const float *__restrict__ route_w, float *__restrict__ out, int rows,
                                                      int slots, int H, int E, int shared_exl3, int e_lo, int e_hi,
                                                      int srow_lo, int srow_hi) {
    // The routing table and the weights were complete before the expert kernels ran (those read them), so they are
    // fetched ahead of the dependency wait; only the pair results Y belong to the kernel in front.
    const int r = blockIdx.y;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    __shared__ float wgt_sh[32];
    __shared__ uint32_t live_sh;
    __shared__ uint32_t used_sh[32];
    if (shared_exl3 == 2) shared_exl3 = shared_owner_of_window(picks, rows * slots, E, e_hi - e_lo, used_sh) == e_lo / (e_hi - e_lo);
    if (threadIdx.x < 32) {
        const int s = threadIdx.x;
        bool keep = false;
        float w = 0.f;
        if (s < slots) {
            const int e = picks[r * slots + s];
            keep = !(e < 0 || e > E || (e == E ? !shared_exl3 : (e < e_lo || e >= e_hi)));
            if (e == E && srow_hi > srow_lo && (r < srow_lo || r >= srow_hi)) keep = false;   // shared expert: row window
            w = route_w[r * slots + s];
        }
        wgt_sh[s] = w;
        const uint32_t mask = __ballot_sync(0xffffffffu, keep);
        if (s == 0) live_sh = mask;
    }
    __syncthreads();
    const uint32_t live = live_sh;
    pdl_wait();
    pdl_launch_dependents();
    if (d >= H) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < slots; ++s) {
        if (!((live >> s) & 1u)) continue;
        const float4 y = *reinterpret_cast<const float4 *>(Y + ((size_t)r * slots + s) * H + d);
        if (s == slots - 1) { acc.x += y.x; acc.y += y.y; acc.z += y.z; acc.w += y.w; }
        else {
            const float w = wgt_sh[s];
            acc.x += w * y.x; acc.y += w * y.y; acc.z += w * y.z; acc.w += w * y.w;
        }
    }
    *reinterpret_cast<float4 *>(out + (size_t)r * H + d) = acc;
}

__global__ void __launch_bounds__(256) rank_sum_kernel(const float *__restrict__ gathered, int world, size_t n,
                                                       float *__restrict__ out) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 acc = *reinterpret_cast<const float4 *>(gathered + i);
    for (int k = 1; k < world; ++k) {
        const float4 v = *reinterpret_cast<const float4 *>(gathered + (size_t)k * n + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4 *>(out + i) = acc;
}

int launch_combine(cudaStream_t s, const float *Y, const int *picks, const float *route_w, float *out, int rows,
                   const glmflash_config &c) {
    const dim3 grid((unsigned)((c.hidden / 4 + 255) / 256), (unsigned)rows);
    return launch_k(combine_kernel, grid, dim3(256), 0, s, c.pdl != 0, Y, picks, route_w, out, rows, c.slots, c.hidden,
                    c.experts, c.shared_exl3, c.expert_lo, c.expert_hi, c.shared_row_lo, c.shared_row_hi);
}
}  // namespace gf

using namespace gf;

struct glmflash_moe {
    glmflash_config cfg;
    glmflash_grouping *grouping = nullptr;
    glmflash_experts *experts = nullptr;            // windows of <= 16 rows
    glmflash_fast_experts *fast = nullptr;          // chunks of > 16 rows
    float *out = nullptr;
    void *in_dev = nullptr;                         // staging for run_host
    int *picks_dev = nullptr;
    float *w_dev = nullptr;
    int phases = 31;                                // profiling aid, see glmflash_moe_set_phases
    bool one_launch = false;                        // windows of <= 16 rows: the one-launch layer kernel (window.cu)
};

extern "C" int glmflash_moe_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_moe **out) {
    GF_REQUIRE(out != nullptr, "out is null");
    *out = nullptr;
    if (check_config(cfg, cfg_bytes, 8192)) return -1;
    glmflash_moe *m = new (std::nothrow) glmflash_moe();
    GF_REQUIRE(m != nullptr, "out of host memory");
    m->cfg = *cfg;
    int rc = glmflash_grouping_new(cfg, cfg_bytes, &m->grouping);
    if (!rc) rc = cfg->max_rows <= 16 ? glmflash_experts_new(cfg, cfg_bytes, &m->experts)
                                      : glmflash_fast_experts_new(cfg, cfg_bytes, &m->fast);
    const size_t rows = cfg->max_rows;
    if (!rc && cudaMalloc((void **)&m->out, rows * cfg->hidden * 4) != cudaSuccess) rc = fail("cudaMalloc(moe out)");
    if (!rc && cudaMalloc(&m->in_dev, rows * cfg->hidden * 2) != cudaSuccess) rc = fail("cudaMalloc(moe staging)");
    if (!rc && cudaMalloc((void **)&m->picks_dev, rows * cfg->slots * 4) != cudaSuccess) rc = fail("cudaMalloc(moe staging)");
    if (!rc && cudaMalloc((void **)&m->w_dev, rows * cfg->slots * 4) != cudaSuccess) rc = fail("cudaMalloc(moe staging)");
    if (rc) {
        glmflash_moe_free(m);
        return -1;
    }
    cudaMemset(m->out, 0, rows * cfg->hidden * 4);
    // Windows of <= 16 rows: three launches per layer (gate/up, down, combine) by default; GLMFLASH_LAYER_KERNELS=1
    // selects the one-launch layer kernel (window.cu), which measured slower on one GPU (43 vs 28 us per one-token layer)
    const char *env = getenv("GLMFLASH_LAYER_KERNELS");
    m->one_launch = env && env[0] == '1';
    *out = m;
    return 0;
}

extern "C" void glmflash_moe_free(glmflash_moe *m) {
    if (!m) return;
    glmflash_grouping_free(m->grouping);
    glmflash_experts_free(m->experts);
    glmflash_fast_experts_free(m->fast);
    cudaFree(m->out); cudaFree(m->in_dev); cudaFree(m->picks_dev); cudaFree(m->w_dev);
    delete m;
}

extern "C" int glmflash_moe_run(glmflash_moe *m, void *stream, const glmflash_weights *w, const void *input, int x_stride,
                                const int32_t *picks, const float *route_w, int rows) {
    GF_REQUIRE(m && w && input && picks && route_w, "null argument");
    GF_REQUIRE(rows > 0 && rows <= m->cfg.max_rows, "rows outside the scratch bound");
    const float *Y;
    if (m->experts && m->one_launch && m->phases == 31 && experts_window_supported(m->cfg, rows))
        // windows of <= 16 rows: grouping, rotation, both projections, epilogues and the combine in one launch
        return experts_run_window(m->experts, (cudaStream_t)stream, w, input, x_stride, picks, route_w, rows, m->out, nullptr, -1);
    if (m->experts) {
        // the same as three launches: grouping and input rotation happen inside the expert kernels
        if (experts_run_fused(m->experts, (cudaStream_t)stream, w, input, x_stride, picks, rows)) return -1;
        Y = glmflash_experts_y(m->experts);
    } else {
        if ((m->phases & 1) && glmflash_grouping_run(m->grouping, stream, picks, rows)) return -1;
        const int32_t *ids = glmflash_grouping_ids(m->grouping), *count = glmflash_grouping_count(m->grouping),
                      *members = glmflash_grouping_members(m->grouping);
        if (glmflash_fast_experts_run(m->fast, stream, w, input, x_stride, picks, ids, count, members, rows,
                                      m->cfg.max_rows, w->suh_g == w->suh_u))
            return -1;
        Y = glmflash_fast_experts_output(m->fast);
    }
    if (!(m->phases & 16)) return 0;
    return launch_combine((cudaStream_t)stream, Y, picks, route_w, m->out, rows, m->cfg);
}

// Expert-parallel form of glmflash_moe_run.  Windows of <= 16 rows: the layer kernel itself pushes each finished block
// of this rank's partial into every peer's receive slot and adds the ranks' slots in rank order (one launch per
// layer and rank); larger windows: the experts of this rank, then the exchange kernel of the owner.
extern "C" int glmflash_moe_run_ep(glmflash_moe *m, glmflash_ep *ep, void *stream, const glmflash_weights *w, const void *input,
                                   int x_stride, const int32_t *picks, const float *route_w, int rows, int shared_here) {
    GF_REQUIRE(m && ep && w && input && picks && route_w, "null argument");
    GF_REQUIRE(rows > 0 && rows <= m->cfg.max_rows, "rows outside the scratch bound");
    if (m->experts && m->one_launch && experts_window_supported(m->cfg, rows)) {
        WinPeers peers;
        float *result = nullptr;
        if (ep_window_peers(ep, &peers, &result)) return -1;
        GF_REQUIRE(peers.max_rows == m->cfg.max_rows, "the layer owner and the exchange owner were built for different row counts");
        return experts_run_window(m->experts, (cudaStream_t)stream, w, input, x_stride, picks, route_w, rows, result,
                                  peers.world > 1 ? &peers : nullptr, shared_here);
    }
    const int shared = shared_here < 0 ? m->cfg.shared_exl3 : shared_here;
    GF_REQUIRE((shared == 2) == (m->cfg.shared_exl3 == 2),
               "the shared expert's owner is decided per window (2) either by both the layer owner and the call, or by neither");
    const int saved = m->phases;
    m->phases &= ~16;                               // experts only: the combine is the exchange kernel's first step
    const int rc = glmflash_moe_run(m, stream, w, input, x_stride, picks, route_w, rows);
    m->phases = saved;
    if (rc) return -1;
    return glmflash_ep_combine(ep, stream, glmflash_moe_pairs(m), picks, route_w, rows, shared);
}

extern "C" int glmflash_moe_set_phases(glmflash_moe *m, int mask) {
    GF_REQUIRE(m != nullptr, "null argument");
    m->phases = mask;
    if (m->experts) return glmflash_experts_set_phases(m->experts, (mask >> 1) & 7);
    return 0;                                      // prefill pipeline: only grouping (1) and combine (16) are selectable here
}

extern "C" float *glmflash_moe_output(const glmflash_moe *m) { return m ? m->out : nullptr; }
extern "C" const int32_t *glmflash_moe_status(const glmflash_moe *m) {
    if (!m) return nullptr;
    return m->experts ? glmflash_experts_status(m->experts) : glmflash_fast_experts_status(m->fast);
}
extern "C" int glmflash_moe_clear_status(glmflash_moe *m, void *stream) {
    GF_REQUIRE(m != nullptr, "null argument");
    return m->experts ? glmflash_experts_clear_status(m->experts, stream) : glmflash_fast_experts_clear_status(m->fast, stream);
}
extern "C" const float *glmflash_moe_pairs(const glmflash_moe *m) {
    if (!m) return nullptr;
    return m->experts ? glmflash_experts_y(m->experts) : glmflash_fast_experts_output(m->fast);
}

extern "C" int glmflash_moe_run_host(glmflash_moe *m, void *stream, const glmflash_weights *w, const void *input_host,
                                     int x_stride, const int32_t *picks_host, const float *route_w_host, int rows,
                                     float *out_host) {
    GF_REQUIRE(m && w && input_host && picks_host && route_w_host && out_host, "null argument");
    GF_REQUIRE(rows > 0 && rows <= m->cfg.max_rows, "rows outside the scratch bound");
    GF_REQUIRE(x_stride == m->cfg.hidden, "run_host takes densely packed rows (x_stride == hidden)");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t H = m->cfg.hidden, S = m->cfg.slots;
    GF_CUDA(cudaMemcpyAsync(m->in_dev, input_host, (size_t)rows * H * 2, cudaMemcpyHostToDevice, s));
    GF_CUDA(cudaMemcpyAsync(m->picks_dev, picks_host, (size_t)rows * S * 4, cudaMemcpyHostToDevice, s));
    GF_CUDA(cudaMemcpyAsync(m->w_dev, route_w_host, (size_t)rows * S * 4, cudaMemcpyHostToDevice, s));
    if (glmflash_moe_run(m, stream, w, m->in_dev, x_stride, m->picks_dev, m->w_dev, rows)) return -1;
    GF_CUDA(cudaMemcpyAsync(out_host, m->out, (size_t)rows * H * 4, cudaMemcpyDeviceToHost, s));
    GF_CUDA(cudaStreamSynchronize(s));
    return 0;
}

extern "C" int glmflash_rank_sum(void *stream, const float *gathered, int world, int rows, int hidden, float *out) {
    GF_REQUIRE(gathered && out, "null argument");
    GF_REQUIRE(world >= 1 && rows >= 1 && hidden >= 4 && hidden % 4 == 0, "bad shape");
    const size_t n = (size_t)rows * hidden;
    rank_sum_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gathered, world, n, out);
    GF_CUDA(cudaGetLastError());
    return 0;
}
