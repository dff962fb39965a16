// Bit-exact trellis decode of whole tiles (the parity probe of the codebook and the tile layout;
// upstream native/exl3.cu:21-40 <=> src/experts.rs:43-74).
#include "common.cuh"

namespace gf {
// One warp per tile.  Lane L owns weights 8L..8L+7 of the tile: the 16-bit windows of the 1024-bit stream
// that end at bits 32L+4, +8, .., +32, cut from word L and the 12 low bits of word L-1 (circular).
__global__ void __launch_bounds__(256) decode_tiles_kernel(const uint32_t *__restrict__ words, long tiles,
                                                           __half *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long tile = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (tile >= tiles) return;
    const uint32_t w = words[tile * 32 + lane];
    const uint32_t p = __shfl_sync(0xffffffffu, w, (lane + 31) & 31);
    __half *o = out + tile * 256;
    const int t = lane & 3, g = lane >> 2;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t state = __funnelshift_r(w, p, 28 - 4 * j) & 0xffffu;
        const int k = 2 * t + (j & 1) + 8 * ((j >> 1) & 1), n = g + 8 * (j >> 2);
        o[k * 16 + n] = codebook(state);
    }
}
}  // namespace gf

extern "C" int glmflash_exl3_decode(void *stream, const uint32_t *words, int64_t tiles, uint16_t *out) {
    GF_REQUIRE(tiles >= 0 && tiles < ((int64_t)1 << 34), "tile count out of range");
    if (tiles == 0) return 0;                      // an empty input is not an error (and has no pointers)
    GF_REQUIRE(words && out, "null argument");
    gf::decode_tiles_kernel<<<(unsigned)((tiles + 7) / 8), 256, 0, (cudaStream_t)stream>>>(words, (long)tiles, (__half *)out);
    GF_CUDA(cudaGetLastError());
    return 0;
}
