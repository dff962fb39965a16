// Internal layout of the decode / verify owner (the C ABI's opaque glmflash_experts), shared by the translation
// units that launch on its scratch: experts.cu (table-driven run_rows), window.cu (the one-launch layer kernel).
#pragma once
#include "common.cuh"

struct glmflash_experts {
    glmflash_config cfg;
    __half *xg = nullptr, *xu = nullptr, *xd = nullptr;   // rotated inputs [P][H], down-projection inputs [P][I]
    float *y = nullptr;                                   // pair results [P][H] (public)
    int *status = nullptr;
    int phases = 7;                                       // profiling aid: 1 = input rotation, 2 = gate/up, 4 = down
    // one-launch layer kernel (window.cu): split partials, arrival counters / ready words, layer output
    float *z1 = nullptr, *z2 = nullptr;                   // split partials [2][H/128][P][I], [I/128][P][H]
    unsigned *sync = nullptr;
    size_t sync_words = 0;
    float *out = nullptr;                                 // [max_rows][H] combined rows of the last window run
    int sm_count = 0;
};

namespace gf {
int check_config(const glmflash_config *cfg, size_t cfg_bytes, int max_rows_limit);

// Peer-mapped receive areas of the expert-parallel exchange fused into the layer kernel's last step.
constexpr int WIN_MAX_WORLD = 8;
struct WinPeers {
    float *recv[WIN_MAX_WORLD];        // recv[k]: rank k's slots [2][world][max_rows][H]
    unsigned *flags[WIN_MAX_WORLD];    // flags[k]: rank k's arrival words [2][world][max_rows][H / 128]
    unsigned *epoch;                   // this rank's exchange counter (every rank advances its own once per exchange)
    int *status;                       // the exchange owner's status word (peer time-outs)
    int rank, world, max_rows;
    unsigned wait_polls;
};


// The whole layer for a window of <= 16 rows in one launch.  out: [rows][H] fp32.  peers == nullptr: single GPU.
int experts_run_window(glmflash_experts *e, cudaStream_t s, const glmflash_weights *w, const void *input, int x_stride,
                       const int32_t *picks, const float *route_w, int rows, float *out, const WinPeers *peers,
                       int shared_here);
bool experts_window_supported(const glmflash_config &c, int rows);
int ep_window_peers(glmflash_ep *h, WinPeers *out, float **result);
}  // namespace gf
