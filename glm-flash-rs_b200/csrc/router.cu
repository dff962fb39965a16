// Router next to the expert path: logits = x . Wr^T and the sigmoid top-k that produces the routing table the expert
// kernels consume.  Upstream runs precompiled kernels here (_router_part, _router_sum, _topk: call sites src/moe.rs:77-111,
// src/window_ops.rs:159-199) whose source is not published, so the semantics are the benchmark's definition:
//   score = sigmoid(logit); the top-k scores of a row, ties to the lower expert id, in descending order;
//   weight = score / sum of the chosen scores; the row's last slot is the shared expert (id E) with weight 1.
// Selection is done on the logits (sigmoid is monotonic), so it does not depend on the precision of expf.
#include "common.cuh"

namespace gf {

// logits[r][e] = sum_k x[r][k] * wr[e][k]: one warp per (row, group of EPW experts); 16-byte loads, lane-strided
// over K, fp32 accumulation, butterfly-reduced.  EPW = 8 re-uses a loaded piece of the row for eight experts (large
// windows: the work is a small GEMM); EPW = 1 gives every (row, expert) its own warp, so that a window of a few rows
// still spreads over many SMs and all of a warp's loads are in flight at once (one memory round trip).
template <int EPW>
__global__ void __launch_bounds__(256) router_logits_kernel(const __nv_bfloat16 *__restrict__ x, int x_stride,
                                                            const __nv_bfloat16 *__restrict__ wr, int rows, int H, int E,
                                                            float *__restrict__ logits) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = (E + EPW - 1) / EPW;
    const long item = (long)blockIdx.x * 8 + warp;
    if (item >= (long)rows * groups) return;
    const int r = (int)(item / groups), e0 = (int)(item % groups) * EPW;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)r * x_stride);     // 8 bf16 per load
    float acc[EPW];
#pragma unroll
    for (int j = 0; j < EPW; ++j) acc[j] = 0.f;
#pragma unroll 8
    for (int c = lane; c < H / 8; c += 32) {
        const uint4 xv = __ldg(xr + c);
        uint4 wv[EPW];
#pragma unroll
        for (int j = 0; j < EPW; ++j)
            wv[j] = e0 + j < E ? __ldg(reinterpret_cast<const uint4 *>(wr + (size_t)(e0 + j) * H) + c) : make_uint4(0u, 0u, 0u, 0u);
        const __nv_bfloat162 *xp = reinterpret_cast<const __nv_bfloat162 *>(&xv);
        float xf[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) { xf[2 * q] = __bfloat162float(xp[q].x); xf[2 * q + 1] = __bfloat162float(xp[q].y); }
#pragma unroll
        for (int j = 0; j < EPW; ++j) {
            const __nv_bfloat162 *wp = reinterpret_cast<const __nv_bfloat162 *>(&wv[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[j] = fmaf(xf[2 * q], __bfloat162float(wp[q].x), acc[j]);
                acc[j] = fmaf(xf[2 * q + 1], __bfloat162float(wp[q].y), acc[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < EPW; ++j) {
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], m);
        if (lane == 0 && e0 + j < E) logits[(size_t)r * E + e0 + j] = acc[j];
    }
}

// Top-k of one row by one warp: lane l holds the logits of experts l, l + 32, ...; k rounds of a warp arg-max (value
// descending, id ascending), the winner is struck out.  E <= 1024.  `row` may point to shared or global memory.
__device__ __forceinline__ void topk_row(const float *row, int E, int topk, int *picks, float *weights, int lane) {
    constexpr int PER = 32;                          // 1024 / 32
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? row[e] : -INFINITY;
    }
    float sum = 0.f, mine = 0.f;                     // lane j keeps the score of the j-th choice
    for (int t = 0; t < topk; ++t) {
        float best = -INFINITY;
        int bid = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = lane + 32 * j;
            if (e < E && (v[j] > best || (v[j] == best && e < bid))) { best = v[j]; bid = e; }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, m);
            const int oi = __shfl_xor_sync(0xffffffffu, bid, m);
            if (ob > best || (ob == best && oi < bid)) { best = ob; bid = oi; }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (lane + 32 * j == bid) v[j] = -INFINITY;                     // struck out (its owner lane only)
        const float score = 1.f / (1.f + expf(-best));
        sum += score;
        if (lane == t) { mine = score; picks[t] = bid; }
    }
    if (lane < topk) weights[lane] = mine / sum;
    if (lane == 0) { picks[topk] = E; weights[topk] = 1.f; }
}

__global__ void __launch_bounds__(256) topk_kernel(const float *__restrict__ logits, int rows, int E, int topk,
                                                   int *__restrict__ picks, float *__restrict__ weights) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    if (r >= rows) return;
    topk_row(logits + (size_t)r * E, E, topk, picks + (size_t)r * (topk + 1), weights + (size_t)r * (topk + 1), lane);
}

// Small windows: logits and top-k of a row in ONE launch.  CTA = row, 32 warps; warp w computes the logits of experts
// w, w + 32, ... (whole-row dot products, all loads of a warp in flight at once, the summation order of
// router_logits_kernel), leaves them in shared memory (and in `logits`), and warp 0 selects.
__global__ void __launch_bounds__(1024) route_row_kernel(const __nv_bfloat16 *__restrict__ x, int x_stride,
                                                         const __nv_bfloat16 *__restrict__ wr, int H, int E, int topk,
                                                         float *__restrict__ logits, int *__restrict__ picks,
                                                         float *__restrict__ weights) {
    __shared__ float row_sh[1024];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = blockIdx.x;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)r * x_stride);
    for (int e = warp; e < E; e += 32) {
        const uint4 *wrow = reinterpret_cast<const uint4 *>(wr + (size_t)e * H);
        float acc = 0.f;
#pragma unroll 8
        for (int c = lane; c < H / 8; c += 32) {
            const uint4 xv = __ldg(xr + c), wv = __ldg(wrow + c);
            const __nv_bfloat162 *xp = reinterpret_cast<const __nv_bfloat162 *>(&xv);
            const __nv_bfloat162 *wp = reinterpret_cast<const __nv_bfloat162 *>(&wv);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc = fmaf(__bfloat162float(xp[q].x), __bfloat162float(wp[q].x), acc);
                acc = fmaf(__bfloat162float(xp[q].y), __bfloat162float(wp[q].y), acc);
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
        if (lane == 0) { row_sh[e] = acc; logits[(size_t)r * E + e] = acc; }
    }
    __syncthreads();
    if (warp == 0) topk_row(row_sh, E, topk, picks + (size_t)r * (topk + 1), weights + (size_t)r * (topk + 1), lane);
}
}  // namespace gf

using namespace gf;

extern "C" int glmflash_router_logits(void *stream, const uint16_t *x, int x_stride, const uint16_t *wr, int rows, int hidden,
                                      int experts, float *logits, int pdl) {
    GF_REQUIRE(x && wr && logits, "null argument");
    GF_REQUIRE(rows > 0 && hidden > 0 && hidden % 8 == 0 && experts > 0, "rows, experts positive; hidden a multiple of 8");
    GF_REQUIRE(x_stride >= hidden && x_stride % 8 == 0, "x_stride must be >= hidden and a multiple of 8");
    GF_REQUIRE(((uintptr_t)x | (uintptr_t)wr) % 16 == 0, "x and the router matrix must be 16-byte aligned");
    if (rows >= 64) {
        const long items = (long)rows * ((experts + 7) / 8);
        return launch_k(router_logits_kernel<8>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, pdl != 0,
                        (const __nv_bfloat16 *)x, x_stride, (const __nv_bfloat16 *)wr, rows, hidden, experts, logits);
    }
    const long items = (long)rows * experts;
    return launch_k(router_logits_kernel<1>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, pdl != 0,
                    (const __nv_bfloat16 *)x, x_stride, (const __nv_bfloat16 *)wr, rows, hidden, experts, logits);
}

extern "C" int glmflash_topk(void *stream, const float *logits, int rows, int experts, int topk, int32_t *picks, float *weights,
                             int pdl) {
    GF_REQUIRE(logits && picks && weights, "null argument");
    GF_REQUIRE(rows > 0 && experts > 0 && experts <= 1024, "experts must be in 1..1024");
    GF_REQUIRE(topk >= 1 && topk <= 31 && topk <= experts, "topk must be in 1..31 and at most the number of experts");
    return launch_k(topk_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, pdl != 0, logits, rows,
                    experts, topk, picks, weights);
}

extern "C" int glmflash_route(void *stream, const uint16_t *x, int x_stride, const uint16_t *wr, int rows, int hidden,
                              int experts, int topk, float *logits, int32_t *picks, float *weights, int pdl) {
    GF_REQUIRE(x && wr && logits && picks && weights, "null argument");
    GF_REQUIRE(rows > 0 && hidden > 0 && hidden % 8 == 0 && experts > 0 && experts <= 1024,
               "rows positive; hidden a multiple of 8; experts in 1..1024");
    GF_REQUIRE(topk >= 1 && topk <= 31 && topk <= experts, "topk must be in 1..31 and at most the number of experts");
    GF_REQUIRE(x_stride >= hidden && x_stride % 8 == 0, "x_stride must be >= hidden and a multiple of 8");
    GF_REQUIRE(((uintptr_t)x | (uintptr_t)wr) % 16 == 0, "x and the router matrix must be 16-byte aligned");
    if (rows <= 16)
        return launch_k(route_row_kernel, dim3((unsigned)rows), dim3(1024), 0, (cudaStream_t)stream, pdl != 0,
                        (const __nv_bfloat16 *)x, x_stride, (const __nv_bfloat16 *)wr, hidden, experts, topk, logits, picks,
                        weights);
    if (glmflash_router_logits(stream, x, x_stride, wr, rows, hidden, experts, logits, pdl)) return -1;
    return glmflash_topk(stream, logits, rows, experts, topk, picks, weights, pdl);
}
