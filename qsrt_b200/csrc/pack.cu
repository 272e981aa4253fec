// Bitstream packer and decoder for trellis tiles (HBM-bound byte work).
//
// A tile's 256 K-bit edge symbols form one MSB-first bitstream of 256*K bits.  The on-disk
// layout is that stream cut into 16-bit words with adjacent words exchanged
// (qsrt/qsrt.py:861-883), which is exactly the stream cut into 32-bit words stored little
// endian.  Both kernels therefore work on whole 32-bit words:
//   pack   : 512 B of states in, 32*K B out per tile, one thread per output word;
//   decode : 32*K B in, 512 B of states and/or 256 B of E4M3 labels out per tile.
// Tiles are staged through shared memory so every global access is coalesced.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

constexpr int kPackTilesPerBlock = 16;
constexpr int kPackThreads = 256;

__global__ void __launch_bounds__(kPackThreads)
pack_kernel(const uint16_t* __restrict__ states, int64_t n_tiles, int bits,
            uint32_t* __restrict__ packed)
{
    __shared__ uint16_t sh[kPackTilesPerBlock * 256];
    const int words_per_tile = 8 * bits;
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t base = int64_t(blockIdx.x) * kPackTilesPerBlock; base < n_tiles;
         base += int64_t(gridDim.x) * kPackTilesPerBlock) {
        const int tiles_here = int(min(int64_t(kPackTilesPerBlock), n_tiles - base));
        // 256 states = 512 B = 32 uint4 per tile
        const uint4* src = reinterpret_cast<const uint4*>(states + base * 256);
        for (int v = threadIdx.x; v < tiles_here * 32; v += kPackThreads)
            reinterpret_cast<uint4*>(sh)[v] = src[v];
        __syncthreads();
        for (int wdx = threadIdx.x; wdx < tiles_here * words_per_tile; wdx += kPackThreads) {
            const int tile = wdx / words_per_tile;
            const int j = wdx - tile * words_per_tile;
            const int bit0 = 32 * j;
            const int s0 = bit0 / bits;
            const int off = bit0 - s0 * bits;
            const int count = (off + 32 + bits - 1) / bits;
            const uint16_t* st = sh + tile * 256 + s0;
            unsigned long long acc = 0;
            for (int s = 0; s < count; ++s) acc = (acc << bits) | (st[s] & mask);
            const int excess = count * bits - off - 32;
            packed[(base + tile) * words_per_tile + j] = uint32_t(acc >> excess);
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256)
unpack_decode_kernel(const uint32_t* __restrict__ packed, int64_t n_tiles, int bits,
                     const uint8_t* __restrict__ lut_state, uint16_t* __restrict__ out_states,
                     uint8_t* __restrict__ out_e4m3)
{
    __shared__ uint32_t words[33];
    __shared__ uint16_t edges[256];
    const int words_per_tile = 8 * bits;
    const uint32_t mask = (1u << bits) - 1u;
    const int lags = (16 + bits - 1) / bits;
    const int i = threadIdx.x;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        if (i < words_per_tile) words[i] = packed[tile * words_per_tile + i];
        if (i == words_per_tile) words[i] = 0;
        __syncthreads();
        const int bit0 = i * bits;
        const int j = bit0 >> 5;
        const int off = bit0 & 31;
        const unsigned long long two = (static_cast<unsigned long long>(words[j]) << 32) | words[j + 1];
        edges[i] = uint16_t((two >> (64 - off - bits)) & mask);
        __syncthreads();
        uint32_t state = 0;
        for (int lag = 0; lag < lags; ++lag) state |= uint32_t(edges[(i - lag) & 255]) << (lag * bits);
        state &= 0xffffu;
        if (out_states) out_states[tile * 256 + i] = uint16_t(state);
        if (out_e4m3) out_e4m3[tile * 256 + i] = lut_state[state];
        __syncthreads();
    }
}

// states [kt, nt, 256] (tensor-core order) -> row-major float32 [kt*16, nt*16].
// One block per tile; thread = row-major element, so the stores of a tile are 16 runs of 64 B.
__global__ void __launch_bounds__(256)
states_to_matrix_kernel(const uint16_t* __restrict__ states, int64_t n_tiles, int tiles_n,
                        const uint8_t* __restrict__ lut_state, float* __restrict__ out, int ld)
{
    __shared__ uint16_t sh[256];
    const int e = threadIdx.x;  // row-major element: row = e / 16, col = e % 16
    const int row = e >> 4, col = e & 15;
    // position of (row, col) in tensor-core order (inverse of exl3_encoder_backend.py:35-57)
    const int lane = ((col & 7) << 2) | ((row & 7) >> 1);
    const int j = (row & 1) | ((row & 8) ? 2 : 0) | ((col & 8) ? 4 : 0);
    const int src = lane * 8 + j;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        sh[e] = states[tile * 256 + e];
        __syncthreads();
        const uint8_t b = lut_state[sh[src]];
        const int64_t tk = tile / tiles_n;
        const int tn = int(tile - tk * tiles_n);
        // E4M3 -> float: exact, via the bit pattern
        const int ex = (b >> 3) & 15, m = b & 7;
        float v = ex == 0 ? float(m) * 0.001953125f : __int_as_float(((ex + 120) << 23) | (m << 20));
        if (b & 0x80) v = -v;
        out[(tk * 16 + row) * int64_t(ld) + tn * 16 + col] = v;
        __syncthreads();
    }
}

int grid_for(int64_t blocks_wanted)
{
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int64_t cap = int64_t(sms) * 8;
    return int(blocks_wanted < cap ? (blocks_wanted > 0 ? blocks_wanted : 1) : cap);
}

}  // namespace

extern "C" int qsrtb_pack_trellis(const int16_t* states, int64_t n_tiles, int bits,
                                  int16_t* packed, void* stream)
{
    if (bits < 2 || bits > 4) return qsrtb_fail(QSRTB_EINVAL, "bits must be 2, 3 or 4");
    if (n_tiles < 0) return qsrtb_fail(QSRTB_EINVAL, "negative tile count");
    if (n_tiles == 0) return QSRTB_OK;
    if (!states || !packed) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    const int64_t blocks = (n_tiles + kPackTilesPerBlock - 1) / kPackTilesPerBlock;
    pack_kernel<<<grid_for(blocks), kPackThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint16_t*>(states), n_tiles, bits, reinterpret_cast<uint32_t*>(packed));
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "pack launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_unpack_decode(const int16_t* packed, int64_t n_tiles, int bits,
                                   const uint8_t* lut_state, int16_t* out_states,
                                   uint8_t* out_e4m3, void* stream)
{
    if (bits < 2 || bits > 4) return qsrtb_fail(QSRTB_EINVAL, "bits must be 2, 3 or 4");
    if (n_tiles < 0) return qsrtb_fail(QSRTB_EINVAL, "negative tile count");
    if (n_tiles == 0) return QSRTB_OK;
    if (!packed || (!out_states && !out_e4m3)) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if (out_e4m3 && !lut_state) return qsrtb_fail(QSRTB_EINVAL, "decoding needs the table");
    unpack_decode_kernel<<<grid_for(n_tiles), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint32_t*>(packed), n_tiles, bits, lut_state,
        reinterpret_cast<uint16_t*>(out_states), out_e4m3);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "unpack launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_states_to_matrix(const int16_t* states, int tiles_k, int tiles_n,
                                      const uint8_t* lut_state, float* out, int ld, void* stream)
{
    if (tiles_k < 0 || tiles_n < 0 || ld < tiles_n * 16) return qsrtb_fail(QSRTB_EINVAL, "bad tile grid");
    const int64_t n_tiles = int64_t(tiles_k) * tiles_n;
    if (n_tiles == 0) return QSRTB_OK;
    if (!states || !lut_state || !out) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    states_to_matrix_kernel<<<grid_for(n_tiles), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint16_t*>(states), n_tiles, tiles_n, lut_state, out, ld);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "states_to_matrix launch");
    return QSRTB_OK;
}
