// Bitstream packer and decoder for trellis tiles (HBM-bound byte work).
//
// A tile's 256 K-bit edge symbols form one MSB-first bitstream of 256*K bits.  The on-disk
// layout is that stream cut into 16-bit words with adjacent words exchanged
// (qsrt/qsrt.py:861-883), which is exactly the stream cut into 32-bit words stored little
// endian.  Both kernels therefore work on whole 32-bit words:
//   pack   : 512 B of states in, 32*K B out per tile, one thread per output word;
//   decode : 32*K B in, 512 B of states and/or 256 B of E4M3 labels out per tile.
// One warp handles one tile: a lane owns 8 consecutive symbols (one 16-byte load or store) and
// exchanges bit chunks with its neighbours through warp shuffles; no shared memory.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

constexpr int kWarpsPerBlock = 8;  // one warp per tile, no shared memory, no block barriers

// A lane owns 8 consecutive symbols = 8*bits (16 / 24 / 32) bits of the tile's bitstream.
__device__ __forceinline__ uint32_t lane_chunk(const uint4 v, int bits)
{
    const uint32_t mask = (1u << bits) - 1u;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t chunk = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        chunk = (chunk << bits) | (w[i] & mask);          // even symbol: low half-word
        chunk = (chunk << bits) | ((w[i] >> 16) & mask);  // odd symbol: high half-word
    }
    return chunk;
}

// Output word `lane` of a tile's packed path from the lanes' 8-symbol chunks.
__device__ __forceinline__ uint32_t packed_word(uint32_t chunk, int lane, int chunk_bits)
{
    // word `lane` starts at bit 32*lane = chunk a, offset off inside chunks a, a+1
    const int a = (32 * lane) / chunk_bits;
    const int off = 32 * lane - a * chunk_bits;
    const uint32_t ca = __shfl_sync(0xffffffffu, chunk, a & 31);
    const uint32_t cb = __shfl_sync(0xffffffffu, chunk, (a + 1) & 31);
    const unsigned long long both = (static_cast<unsigned long long>(ca) << chunk_bits) | cb;
    return uint32_t(both >> (2 * chunk_bits - off - 32));
}

// Two tiles per warp and iteration: both 512-byte loads are issued before either is consumed,
// which doubles the bytes in flight per SM.
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
pack_kernel(const uint16_t* __restrict__ states, int64_t n_tiles, int bits,
            uint32_t* __restrict__ packed)
{
    const int lane = threadIdx.x & 31;
    const int chunk_bits = 8 * bits;
    const int words_per_tile = 8 * bits;
    const int64_t stride = int64_t(gridDim.x) * kWarpsPerBlock;
    for (int64_t tile = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); tile < n_tiles;
         tile += 2 * stride) {
        const int64_t other = tile + stride;
        const bool pair = other < n_tiles;
        const uint4 v0 = reinterpret_cast<const uint4*>(states + tile * 256)[lane];
        const uint4 v1 = pair ? reinterpret_cast<const uint4*>(states + other * 256)[lane] : make_uint4(0, 0, 0, 0);
        const uint32_t w0 = packed_word(lane_chunk(v0, bits), lane, chunk_bits);
        const uint32_t w1 = packed_word(lane_chunk(v1, bits), lane, chunk_bits);
        if (lane < words_per_tile) {
            packed[tile * words_per_tile + lane] = w0;
            if (pair) packed[other * words_per_tile + lane] = w1;
        }
    }
}

__global__ void __launch_bounds__(32 * kWarpsPerBlock)
unpack_decode_kernel(const uint32_t* __restrict__ packed, int64_t n_tiles, int bits,
                     const uint8_t* __restrict__ lut_state, uint16_t* __restrict__ out_states,
                     uint8_t* __restrict__ out_e4m3)
{
    extern __shared__ __align__(16) uint8_t sh_lut[];  // 64 KiB copy of the table when decoding
    if (out_e4m3) {
        const uint4* src = reinterpret_cast<const uint4*>(lut_state);
        for (int i = threadIdx.x; i < 4096; i += blockDim.x) reinterpret_cast<uint4*>(sh_lut)[i] = src[i];
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int chunk_bits = 8 * bits;
    const int words_per_tile = 8 * bits;
    const unsigned long long chunk_mask = (1ull << chunk_bits) - 1ull;
    for (int64_t tile = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); tile < n_tiles;
         tile += int64_t(gridDim.x) * kWarpsPerBlock) {
        const uint32_t* words = packed + tile * words_per_tile;
        const int bit0 = lane * chunk_bits;
        const int w = bit0 >> 5, off = bit0 & 31;
        const uint32_t w0 = words[w];
        const uint32_t w1 = words[min(w + 1, words_per_tile - 1)];
        const unsigned long long two = (static_cast<unsigned long long>(w0) << 32) | w1;
        const uint32_t chunk = uint32_t((two >> (64 - off - chunk_bits)) & chunk_mask);
        // the 8 symbols before this lane's (cyclic) complete every 16-bit state window
        const uint32_t prev = __shfl_sync(0xffffffffu, chunk, (lane + 31) & 31);
        const unsigned long long window = (static_cast<unsigned long long>(prev) << chunk_bits) | chunk;
        uint32_t st[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) st[i] = uint32_t(window >> ((7 - i) * bits)) & 0xffffu;
        if (out_states) {
            const uint4 v = make_uint4(st[0] | (st[1] << 16), st[2] | (st[3] << 16),
                                       st[4] | (st[5] << 16), st[6] | (st[7] << 16));
            reinterpret_cast<uint4*>(out_states + tile * 256)[lane] = v;
        }
        if (out_e4m3) {
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lo |= uint32_t(sh_lut[st[i]]) << (8 * i);
                hi |= uint32_t(sh_lut[st[4 + i]]) << (8 * i);
            }
            reinterpret_cast<uint2*>(out_e4m3 + tile * 256)[lane] = make_uint2(lo, hi);
        }
    }
}

// States only (no table): two tiles per warp and iteration, both loads issued before the first
// shuffle, so that a warp keeps two independent 512-byte stores behind one load latency.
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
unpack_states_kernel(const uint32_t* __restrict__ packed, int64_t n_tiles, int bits, uint16_t* __restrict__ out_states)
{
    const int lane = threadIdx.x & 31;
    const int chunk_bits = 8 * bits, words_per_tile = 8 * bits;
    const unsigned long long chunk_mask = (1ull << chunk_bits) - 1ull;
    const int bit0 = lane * chunk_bits;
    const int w = bit0 >> 5, off = bit0 & 31;
    const int w_next = min(w + 1, words_per_tile - 1);
    const int64_t warps = int64_t(gridDim.x) * kWarpsPerBlock;
    const int64_t pairs = (n_tiles + 1) / 2;
    for (int64_t pair = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); pair < pairs; pair += warps) {
        uint32_t w0[2], w1[2];
        bool live[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int64_t tile = 2 * pair + u;
            live[u] = tile < n_tiles;
            const uint32_t* words = packed + (live[u] ? tile : 0) * words_per_tile;
            w0[u] = words[w];
            w1[u] = words[w_next];
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const unsigned long long two = (static_cast<unsigned long long>(w0[u]) << 32) | w1[u];
            const uint32_t chunk = uint32_t((two >> (64 - off - chunk_bits)) & chunk_mask);
            const uint32_t prev = __shfl_sync(0xffffffffu, chunk, (lane + 31) & 31);
            const unsigned long long window = (static_cast<unsigned long long>(prev) << chunk_bits) | chunk;
            uint32_t st[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) st[i] = uint32_t(window >> ((7 - i) * bits)) & 0xffffu;
            if (live[u])
                reinterpret_cast<uint4*>(out_states + (2 * pair + u) * 256)[lane] =
                    make_uint4(st[0] | (st[1] << 16), st[2] | (st[3] << 16), st[4] | (st[5] << 16), st[6] | (st[7] << 16));
        }
    }
}

// Labels only: 32 warps per SM share one staged copy of the table (one 1024-thread CTA per SM) and
// every warp decodes two tiles per iteration, so two tiles' loads and their 16 table look-ups per
// lane are in flight together; with one tile per warp the kernel waited on its own load latency.
__global__ void __launch_bounds__(1024, 1)
decode_e4m3_kernel(const uint32_t* __restrict__ packed, int64_t n_tiles, int bits,
                   const uint8_t* __restrict__ lut_state, uint8_t* __restrict__ out_e4m3)
{
    extern __shared__ __align__(16) uint8_t sh_lut[];
    {
        const uint4* src = reinterpret_cast<const uint4*>(lut_state);
        for (int i = threadIdx.x; i < 4096; i += blockDim.x) reinterpret_cast<uint4*>(sh_lut)[i] = src[i];
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int chunk_bits = 8 * bits, words_per_tile = 8 * bits;
    const unsigned long long chunk_mask = (1ull << chunk_bits) - 1ull;
    const int bit0 = lane * chunk_bits;
    const int w = bit0 >> 5, off = bit0 & 31;
    const int w_next = min(w + 1, words_per_tile - 1);
    const int64_t warps = int64_t(gridDim.x) * 32;
    const int64_t pairs = (n_tiles + 1) / 2;
    for (int64_t pair = int64_t(blockIdx.x) * 32 + (threadIdx.x >> 5); pair < pairs; pair += warps) {
        uint32_t w0[2], w1[2];
        bool live[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int64_t tile = 2 * pair + u;
            live[u] = tile < n_tiles;
            const uint32_t* words = packed + (live[u] ? tile : 0) * words_per_tile;
            w0[u] = words[w];
            w1[u] = words[w_next];
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const unsigned long long two = (static_cast<unsigned long long>(w0[u]) << 32) | w1[u];
            const uint32_t chunk = uint32_t((two >> (64 - off - chunk_bits)) & chunk_mask);
            const uint32_t prev = __shfl_sync(0xffffffffu, chunk, (lane + 31) & 31);
            const unsigned long long window = (static_cast<unsigned long long>(prev) << chunk_bits) | chunk;
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lo |= uint32_t(sh_lut[uint32_t(window >> ((7 - i) * bits)) & 0xffffu]) << (8 * i);
                hi |= uint32_t(sh_lut[uint32_t(window >> ((3 - i) * bits)) & 0xffffu]) << (8 * i);
            }
            if (live[u]) reinterpret_cast<uint2*>(out_e4m3 + (2 * pair + u) * 256)[lane] = make_uint2(lo, hi);
        }
    }
}

// states [kt, nt, 256] (tensor-core order) -> row-major float32 [kt*16, nt*16].
// One warp per tile.  Lane l holds tensor-core elements 8l..8l+7, i.e. rows {r0, r0+1, r0+8,
// r0+9} x columns {c0, c0+8} with r0 = 2*(l%4), c0 = l/4 (exl3_encoder_backend.py:35-57): each
// of its 8 stores lands in a run of 8 consecutive floats shared with 7 other lanes.
// One 1024-thread CTA per SM stages the table once; a warp takes two tiles per iteration so that
// both 512-byte loads are in flight before the first look-up.
__global__ void __launch_bounds__(1024, 1)
states_to_matrix_kernel(const uint16_t* __restrict__ states, int64_t n_tiles, int tiles_n,
                        const uint8_t* __restrict__ lut_state, float* __restrict__ out, int ld)
{
    extern __shared__ __align__(16) uint8_t sh_lut[];
    {
        const uint4* src = reinterpret_cast<const uint4*>(lut_state);
        for (int i = threadIdx.x; i < 4096; i += blockDim.x) reinterpret_cast<uint4*>(sh_lut)[i] = src[i];
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int r0 = (lane & 3) * 2, c0 = lane >> 2;
    const int64_t warps = int64_t(gridDim.x) * 32;
    const int64_t pairs = (n_tiles + 1) / 2;
    for (int64_t pair = int64_t(blockIdx.x) * 32 + (threadIdx.x >> 5); pair < pairs; pair += warps) {
        uint4 v[2];
        bool live[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int64_t tile = 2 * pair + u;
            live[u] = tile < n_tiles;
            v[u] = reinterpret_cast<const uint4*>(states + (live[u] ? tile : 0) * 256)[lane];
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!live[u]) continue;
            const int64_t tile = 2 * pair + u;
            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
            const int64_t tk = tile / tiles_n;
            const int tn = int(tile - tk * tiles_n);
            float* base = out + (tk * 16) * int64_t(ld) + tn * 16;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t state = (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu);
                const uint8_t b = sh_lut[state];
                // E4M3 -> float: exact, via the bit pattern
                const int ex = (b >> 3) & 15, m = b & 7;
                float value = ex == 0 ? float(m) * 0.001953125f : __int_as_float(((ex + 120) << 23) | (m << 20));
                if (b & 0x80) value = -value;
                const int row = r0 + (j & 1) + ((j & 2) ? 8 : 0);
                const int col = c0 + ((j & 4) ? 8 : 0);
                base[int64_t(row) * ld + col] = value;
            }
        }
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

// Kernels that stage the 64 KiB table in shared memory run three blocks per SM and loop.
int lut_grid(int64_t n_tiles)
{
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int64_t wanted = (n_tiles + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int64_t cap = int64_t(sms) * 3;
    return int(wanted < cap ? (wanted > 0 ? wanted : 1) : cap);
}

}  // namespace

extern "C" int qsrtb_pack_trellis(const int16_t* states, int64_t n_tiles, int bits,
                                  int16_t* packed, void* stream)
{
    if (bits < 2 || bits > 4) return qsrtb_fail(QSRTB_EINVAL, "bits must be 2, 3 or 4");
    if (n_tiles < 0) return qsrtb_fail(QSRTB_EINVAL, "negative tile count");
    if (n_tiles == 0) return QSRTB_OK;
    if (!states || !packed) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    const int64_t blocks = (n_tiles + kWarpsPerBlock - 1) / kWarpsPerBlock;
    pack_kernel<<<grid_for(blocks), 32 * kWarpsPerBlock, 0, static_cast<cudaStream_t>(stream)>>>(
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
    if (out_e4m3 && !out_states) {
        int device = 0, sms = 148;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        const int64_t wanted = (n_tiles + 63) / 64;   // 32 warps x 2 tiles per block and iteration
        cudaFuncSetAttribute(decode_e4m3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
        decode_e4m3_kernel<<<int(wanted < sms ? wanted : sms), 1024, 65536, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const uint32_t*>(packed), n_tiles, bits, lut_state, out_e4m3);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return qsrtb_fail_cuda(e, "decode launch");
        return QSRTB_OK;
    }
    if (out_states && !out_e4m3) {
        unpack_states_kernel<<<grid_for((n_tiles + 2 * kWarpsPerBlock - 1) / (2 * kWarpsPerBlock)), 32 * kWarpsPerBlock, 0,
                               static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const uint32_t*>(packed), n_tiles, bits, reinterpret_cast<uint16_t*>(out_states));
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return qsrtb_fail_cuda(e, "unpack launch");
        return QSRTB_OK;
    }
    const size_t smem = out_e4m3 ? 65536 : 0;
    cudaFuncSetAttribute(unpack_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    const int grid = out_e4m3 ? lut_grid(n_tiles) : grid_for((n_tiles + kWarpsPerBlock - 1) / kWarpsPerBlock);
    unpack_decode_kernel<<<grid, 32 * kWarpsPerBlock, smem, static_cast<cudaStream_t>(stream)>>>(
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
    cudaFuncSetAttribute(states_to_matrix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int64_t wanted = (n_tiles + 63) / 64;   // 32 warps x 2 tiles per block and iteration
    states_to_matrix_kernel<<<int(wanted < sms ? wanted : sms), 1024, 65536, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint16_t*>(states), n_tiles, tiles_n, lut_state, out, ld);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "states_to_matrix launch");
    return QSRTB_OK;
}
