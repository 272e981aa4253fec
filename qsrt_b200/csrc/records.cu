// Mixed-rate record container and atom-major storage image (HBM-bound byte work).
//
// A complete expert matrix is cut along its rate axis into records of `stripes` tile rows (or
// tile columns); every record has its own edge width K in {2,3,4}.  Two destination layouts:
//
//   records : the records' packed tiles, record after record, tiles inside a record in
//             row-major tile order (qsrt/qsrt.py:1051-1082);
//   atoms   : atom (pair p, stripe s) holds stripe s of record 2p followed by stripe s of record
//             2p+1; atom a is stored in slot (a + rotation) mod n_atoms at a fixed byte pitch,
//             which lets three matrices and their scales share one bundle per slot
//             (qsrt/qsrt_storage.py:194-231,347-362,441-462).
//
// One warp per tile: it reads the tile's 512 bytes of states in one piece and writes one
// contiguous run of 32*K bytes; a block row covers one tile row (column) of the rate axis, so the
// record, its width and its offset are derived once per block and no index needs a division.  Nothing is materialised in between:
// states -> final image is one read of the states and one write of the image.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxRecords = 64;

struct RecordLayout {
    int tiles_k, tiles_n;
    int rate_axis;      // 0: records cut the K (row) axis, 1: the N (column) axis
    int n_records;
    int stripes;        // tile rows (columns) per record
    int orth;           // tiles along the other axis
    int layout;         // 0 records, 1 atoms
    int rotation;       // atoms: slot = (atom + rotation) mod n_atoms
    int64_t atom_pitch32;             // atoms: 32-bit words between consecutive slots
    uint8_t bits[kMaxRecords];
    int64_t record_off32[kMaxRecords];  // records: first 32-bit word of each record
};

struct Placement {
    int64_t src_tile;   // index into [tiles_k, tiles_n]
    int64_t dst32;      // first 32-bit word of the tile's packed path
    int bits;
};

// Tile `o` (position along the orthogonal axis) of tile row/column `along` of the rate axis.
// The grid's y index is `along`, so a block derives record and stripe once and its warps step
// through `o` without any division.
__device__ __forceinline__ Placement place(const RecordLayout& g, int along, int o)
{
    Placement p;
    const int record = along / g.stripes;
    const int stripe = along - record * g.stripes;
    p.bits = g.bits[record];
    if (g.layout == 0) {
        const int idx = g.rate_axis == 0 ? stripe * g.orth + o : o * g.stripes + stripe;
        p.dst32 = g.record_off32[record] + int64_t(idx) * 8 * p.bits;
    } else {
        const int pair = record >> 1, side = record & 1;
        const int n_atoms = (g.n_records / 2) * g.stripes;
        int slot = pair * g.stripes + stripe + g.rotation;
        if (slot >= n_atoms) slot -= n_atoms;
        p.dst32 = int64_t(slot) * g.atom_pitch32 + (side ? int64_t(g.orth) * 8 * g.bits[2 * pair] : 0) +
                  int64_t(o) * 8 * p.bits;
    }
    p.src_tile = g.rate_axis == 0 ? int64_t(along) * g.tiles_n + o : int64_t(o) * g.tiles_n + along;
    return p;
}

// A lane owns 8 consecutive symbols = 8*bits bits of the tile's MSB-first bitstream.
__device__ __forceinline__ uint32_t lane_chunk(const uint4 v, int bits)
{
    const uint32_t mask = (1u << bits) - 1u;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t chunk = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        chunk = (chunk << bits) | (w[i] & mask);
        chunk = (chunk << bits) | ((w[i] >> 16) & mask);
    }
    return chunk;
}

// The 8 states of a lane from its own chunk and the (cyclically) previous lane's.
__device__ __forceinline__ void lane_states(uint32_t chunk, uint32_t prev, int bits, uint32_t st[8])
{
    const unsigned long long window = (static_cast<unsigned long long>(prev) << (8 * bits)) | chunk;
#pragma unroll
    for (int i = 0; i < 8; ++i) st[i] = uint32_t(window >> ((7 - i) * bits)) & 0xffffu;
}

// Packs one tile held as a lane-distributed uint4 and, when asked, counts it if it is not a closed
// cyclic walk: every 16-bit state must equal the window of the last ceil(16/K) edge symbols
// (qsrt/qsrt.py:1074-1078).
__device__ __forceinline__ void pack_one(const uint4 v, const Placement& p, int lane, uint32_t* __restrict__ dst,
                                         int* __restrict__ open_paths)
{
    const int chunk_bits = 8 * p.bits;
    const uint32_t chunk = lane_chunk(v, p.bits);
    if (open_paths) {
        const uint32_t prev = __shfl_sync(0xffffffffu, chunk, (lane + 31) & 31);
        uint32_t st[8];
        lane_states(chunk, prev, p.bits, st);
        const bool same = v.x == (st[0] | (st[1] << 16)) && v.y == (st[2] | (st[3] << 16)) &&
                          v.z == (st[4] | (st[5] << 16)) && v.w == (st[6] | (st[7] << 16));
        const unsigned bad = __ballot_sync(0xffffffffu, !same);
        if (bad && lane == 0) atomicAdd(open_paths, 1);
    }
    const int a = (32 * lane) / chunk_bits;
    const int off = 32 * lane - a * chunk_bits;
    const uint32_t ca = __shfl_sync(0xffffffffu, chunk, a & 31);
    const uint32_t cb = __shfl_sync(0xffffffffu, chunk, (a + 1) & 31);
    const unsigned long long both = (static_cast<unsigned long long>(ca) << chunk_bits) | cb;
    const uint32_t word = uint32_t(both >> (2 * chunk_bits - off - 32));
    if (lane < chunk_bits) dst[p.dst32 + lane] = word;
}

// Two tiles per warp and iteration: both 512-byte loads are issued before either is consumed.
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
pack_records_kernel(const uint16_t* __restrict__ states, int64_t n_tiles, RecordLayout g,
                    uint32_t* __restrict__ dst, int* __restrict__ open_paths)
{
    const int lane = threadIdx.x & 31;
    const int stride = gridDim.x * kWarpsPerBlock;
    for (int o = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); o < g.orth; o += 2 * stride) {
        const bool pair = o + stride < g.orth;
        const Placement p0 = place(g, blockIdx.y, o);
        const Placement p1 = place(g, blockIdx.y, pair ? o + stride : o);
        const uint4 v0 = reinterpret_cast<const uint4*>(states + p0.src_tile * 256)[lane];
        const uint4 v1 = reinterpret_cast<const uint4*>(states + p1.src_tile * 256)[lane];
        pack_one(v0, p0, lane, dst, open_paths);
        if (pair) pack_one(v1, p1, lane, dst, open_paths);
    }
}

__global__ void __launch_bounds__(32 * kWarpsPerBlock)
unpack_records_kernel(const uint32_t* __restrict__ src, int64_t n_tiles, RecordLayout g,
                      uint16_t* __restrict__ out_states, uint16_t* __restrict__ out_edges)
{
    const int lane = threadIdx.x & 31;
    for (int o = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); o < g.orth; o += gridDim.x * kWarpsPerBlock) {
        const Placement p = place(g, blockIdx.y, o);
        const int chunk_bits = 8 * p.bits;
        const uint32_t* words = src + p.dst32;
        const int bit0 = lane * chunk_bits;
        const int w = bit0 >> 5, off = bit0 & 31;
        const uint32_t w0 = words[w];
        const uint32_t w1 = words[min(w + 1, chunk_bits - 1)];
        const unsigned long long two = (static_cast<unsigned long long>(w0) << 32) | w1;
        const uint32_t chunk = uint32_t((two >> (64 - off - chunk_bits)) & ((1ull << chunk_bits) - 1ull));
        const uint32_t prev = __shfl_sync(0xffffffffu, chunk, (lane + 31) & 31);
        uint32_t st[8];
        lane_states(chunk, prev, p.bits, st);
        if (out_states) {
            reinterpret_cast<uint4*>(out_states + p.src_tile * 256)[lane] =
                make_uint4(st[0] | (st[1] << 16), st[2] | (st[3] << 16), st[4] | (st[5] << 16),
                           st[6] | (st[7] << 16));
        }
        if (out_edges) {
            const uint32_t m = (1u << p.bits) - 1u;
            reinterpret_cast<uint4*>(out_edges + p.src_tile * 256)[lane] =
                make_uint4((st[0] & m) | ((st[1] & m) << 16), (st[2] & m) | ((st[3] & m) << 16),
                           (st[4] & m) | ((st[5] & m) << 16), (st[6] & m) | ((st[7] & m) << 16));
        }
    }
}

// Packed tile paths between the two layouts, without touching the bits: warp per tile, walking
// atom order; lane l moves 32-bit word l of the path.
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
records_atoms_kernel(uint32_t* __restrict__ records, int64_t n_tiles, RecordLayout g_records,
                     RecordLayout g_atoms, uint32_t* __restrict__ atoms, int to_records)
{
    const int lane = threadIdx.x & 31;
    for (int o = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); o < g_atoms.orth;
         o += gridDim.x * kWarpsPerBlock) {
        const Placement pa = place(g_atoms, blockIdx.y, o);
        const int64_t rec32 = place(g_records, blockIdx.y, o).dst32;
        if (lane < 8 * pa.bits) {
            if (to_records) records[rec32 + lane] = atoms[pa.dst32 + lane];
            else atoms[pa.dst32 + lane] = records[rec32 + lane];
        }
    }
}

// grid.y = tile rows (columns) along the rate axis, grid.x covers the orthogonal tiles.
dim3 grid_for(const RecordLayout& g)
{
    const int along = g.n_records * g.stripes;
    // each warp takes two tiles per iteration
    return dim3(unsigned((g.orth + 2 * kWarpsPerBlock - 1) / (2 * kWarpsPerBlock)), unsigned(along));
}

// Validates the geometry and fills the layout; returns the bytes the destination must hold.
int make_layout(int tiles_k, int tiles_n, int rate_axis, int n_records, int stripes,
                const uint8_t* record_bits, int layout, int rotation, int64_t atom_pitch_bytes,
                RecordLayout* g, int64_t* extent_bytes)
{
    if (tiles_k <= 0 || tiles_n <= 0) return qsrtb_fail(QSRTB_EINVAL, "tile grid must be positive");
    if (int64_t(tiles_k) * tiles_n > (int64_t(1) << 30)) return qsrtb_fail(QSRTB_EINVAL, "tile grid too large");
    if (rate_axis != 0 && rate_axis != 1) return qsrtb_fail(QSRTB_EINVAL, "rate_axis must be 0 (k) or 1 (n)");
    if (n_records <= 0 || n_records > kMaxRecords || stripes <= 0 || !record_bits)
        return qsrtb_fail(QSRTB_EINVAL, "bad record description");
    const int along = rate_axis == 0 ? tiles_k : tiles_n;
    if (int64_t(n_records) * stripes != along)
        return qsrtb_fail(QSRTB_EINVAL, "records do not cover the rate axis");
    if (along > 65535) return qsrtb_fail(QSRTB_EINVAL, "rate axis longer than 65535 tiles");
    g->tiles_k = tiles_k; g->tiles_n = tiles_n; g->rate_axis = rate_axis;
    g->n_records = n_records; g->stripes = stripes;
    g->orth = rate_axis == 0 ? tiles_n : tiles_k;
    g->layout = layout; g->rotation = 0; g->atom_pitch32 = 0;
    int64_t cursor = 0;
    for (int r = 0; r < n_records; ++r) {
        const int b = record_bits[r];
        if (b < 2 || b > 4) return qsrtb_fail(QSRTB_EINVAL, "record bits must be 2, 3 or 4");
        g->bits[r] = uint8_t(b);
        g->record_off32[r] = cursor;
        cursor += int64_t(stripes) * g->orth * 8 * b;
    }
    if (layout == 0) {
        *extent_bytes = cursor * 4;
        return QSRTB_OK;
    }
    if (layout != 1) return qsrtb_fail(QSRTB_EINVAL, "layout must be 0 (records) or 1 (atoms)");
    if (n_records % 2) return qsrtb_fail(QSRTB_EINVAL, "atoms need an even record count");
    const int n_atoms = (n_records / 2) * stripes;
    if (rotation < 0 || rotation >= n_atoms) return qsrtb_fail(QSRTB_EINVAL, "rotation out of range");
    int64_t widest = 0;
    for (int p = 0; p < n_records / 2; ++p) {
        const int64_t bytes = int64_t(g->orth) * 32 * (g->bits[2 * p] + g->bits[2 * p + 1]);
        widest = bytes > widest ? bytes : widest;
    }
    if (atom_pitch_bytes < widest || (atom_pitch_bytes % 4))
        return qsrtb_fail(QSRTB_EINVAL, "atom pitch must be a multiple of 4 bytes and hold the widest atom");
    g->rotation = rotation;
    g->atom_pitch32 = atom_pitch_bytes / 4;
    *extent_bytes = int64_t(n_atoms - 1) * atom_pitch_bytes + widest;
    return QSRTB_OK;
}

}  // namespace

extern "C" int qsrtb_pack_records(const int16_t* states, int tiles_k, int tiles_n, int rate_axis,
                                  int n_records, int stripes, const uint8_t* record_bits, int layout,
                                  int rotation, int64_t atom_pitch_bytes, int16_t* dst, int64_t dst_bytes,
                                  int* open_paths, void* stream)
{
    RecordLayout g;
    int64_t extent = 0;
    const int rc = make_layout(tiles_k, tiles_n, rate_axis, n_records, stripes, record_bits, layout, rotation,
                               atom_pitch_bytes, &g, &extent);
    if (rc != QSRTB_OK) return rc;
    if (!states || !dst) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if ((reinterpret_cast<uintptr_t>(dst) & 3) || (reinterpret_cast<uintptr_t>(states) & 15))
        return qsrtb_fail(QSRTB_EINVAL, "states need 16-byte and the destination 4-byte alignment");
    if (dst_bytes < extent) return qsrtb_fail(QSRTB_EINVAL, "destination too small for the payload");
    const int64_t n_tiles = int64_t(tiles_k) * tiles_n;
    pack_records_kernel<<<grid_for(g), 32 * kWarpsPerBlock, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint16_t*>(states), n_tiles, g, reinterpret_cast<uint32_t*>(dst), open_paths);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "pack_records launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_unpack_records(const int16_t* src, int64_t src_bytes, int tiles_k, int tiles_n,
                                    int rate_axis, int n_records, int stripes, const uint8_t* record_bits,
                                    int layout, int rotation, int64_t atom_pitch_bytes, int16_t* out_states,
                                    int16_t* out_edges, void* stream)
{
    RecordLayout g;
    int64_t extent = 0;
    const int rc = make_layout(tiles_k, tiles_n, rate_axis, n_records, stripes, record_bits, layout, rotation,
                               atom_pitch_bytes, &g, &extent);
    if (rc != QSRTB_OK) return rc;
    if (!src || (!out_states && !out_edges)) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if ((reinterpret_cast<uintptr_t>(src) & 3) || (reinterpret_cast<uintptr_t>(out_states) & 15) ||
        (reinterpret_cast<uintptr_t>(out_edges) & 15))
        return qsrtb_fail(QSRTB_EINVAL, "outputs need 16-byte and the payload 4-byte alignment");
    if (src_bytes < extent) return qsrtb_fail(QSRTB_EINVAL, "payload shorter than its description");
    const int64_t n_tiles = int64_t(tiles_k) * tiles_n;
    unpack_records_kernel<<<grid_for(g), 32 * kWarpsPerBlock, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint32_t*>(src), n_tiles, g, reinterpret_cast<uint16_t*>(out_states),
        reinterpret_cast<uint16_t*>(out_edges));
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "unpack_records launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_records_atoms(int16_t* records, int64_t records_bytes, int tiles_k, int tiles_n,
                                   int rate_axis, int n_records, int stripes, const uint8_t* record_bits,
                                   int rotation, int64_t atom_pitch_bytes, int16_t* atoms, int64_t atoms_bytes,
                                   int to_records, void* stream)
{
    RecordLayout g_records, g_atoms;
    int64_t extent_records = 0, extent_atoms = 0;
    int rc = make_layout(tiles_k, tiles_n, rate_axis, n_records, stripes, record_bits, 0, 0, 0, &g_records,
                         &extent_records);
    if (rc != QSRTB_OK) return rc;
    rc = make_layout(tiles_k, tiles_n, rate_axis, n_records, stripes, record_bits, 1, rotation, atom_pitch_bytes,
                     &g_atoms, &extent_atoms);
    if (rc != QSRTB_OK) return rc;
    if (!records || !atoms) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if ((reinterpret_cast<uintptr_t>(records) & 3) || (reinterpret_cast<uintptr_t>(atoms) & 3))
        return qsrtb_fail(QSRTB_EINVAL, "payloads need 4-byte alignment");
    if (records_bytes < extent_records || atoms_bytes < extent_atoms)
        return qsrtb_fail(QSRTB_EINVAL, "buffer shorter than its description");
    const int64_t n_tiles = int64_t(tiles_k) * tiles_n;
    records_atoms_kernel<<<grid_for(g_atoms), 32 * kWarpsPerBlock, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<uint32_t*>(records), n_tiles, g_records, g_atoms, reinterpret_cast<uint32_t*>(atoms),
        to_records);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "records_atoms launch");
    return QSRTB_OK;
}
