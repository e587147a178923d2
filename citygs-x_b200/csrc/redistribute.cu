// Row redistribution by a destination vector: the anchor redistribution of the reference
// (scene/gaussian_model.py:1485-1558 all2all_gaussian_state, driven by redistribute_gaussians :1683-1764) as ONE
// packed exchange.  The reference moves every tensor of the model state (parameters, Adam moments, level tags) with
// its own list all-to-all, selecting `state[destination == j]` per destination in Python.  Here all tensors travel
// together: a row of the exchange is the concatenation of the row of every tensor (4-byte words), one kernel counts
// rows per destination, one kernel packs every tensor's rows straight into the destination's segment (the send
// buffer of a collective, or the peer's memory), one kernel splits the received rows back into tensors.
// Order kept from the reference: per destination ascending local index; on the receiver sources ascending.
// Pure data movement: HBM / NVLink bound, bit-exact.
#include "cgx_common.cuh"

namespace cgx {

constexpr int RD_MAX_WS = 32;
constexpr int RD_MAX_TENSORS = 32;
constexpr int RD_TILE = 256;   // rows per CTA

struct RowTensors {
    int n;                              // tensors
    int words[RD_MAX_TENSORS];          // 4-byte words per row of tensor t
    int offset[RD_MAX_TENSORS + 1];     // first word of tensor t inside an exchange row
    void* ptr[RD_MAX_TENSORS];          // (rows, words[t]) arrays
};

struct RowDsts {
    uint32_t* base[RD_MAX_WS];          // destination j's row array (send-buffer segment or peer memory)
    long long first_row[RD_MAX_WS];     // first row this rank writes there
};

// block_counts[j * nblocks + b] = rows of CTA b that go to destination j
__global__ void __launch_bounds__(RD_TILE)
rows_dest_count_kernel(long long n, int ws, int nblocks, const int32_t* __restrict__ destination,
                       uint32_t* __restrict__ block_counts, int* __restrict__ bad)
{
    __shared__ uint32_t s_cnt[RD_MAX_WS];
    if (threadIdx.x < RD_MAX_WS) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    const long long i = (long long)blockIdx.x * RD_TILE + threadIdx.x;
    int d = -1;
    if (i < n) {
        d = destination[i];
        if (d < 0 || d >= ws) {          // a destination outside the group: reported, row dropped
            atomicExch(bad, 1);
            d = -1;
        }
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    if (d >= 0 && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&s_cnt[d], (uint32_t)__popc(peers));
    __syncthreads();
    if (threadIdx.x < ws) block_counts[(size_t)threadIdx.x * nblocks + blockIdx.x] = s_cnt[threadIdx.x];
}

// Every row goes to   base[d] + (first_row[d] + rows of destination d before it on this rank) * row_words,
// tensor after tensor.  The position inside the CTA comes from ballots (stable: ascending row index).
__global__ void __launch_bounds__(RD_TILE)
rows_pack_kernel(long long n, int ws, int nblocks, const int32_t* __restrict__ destination,
                 const uint32_t* __restrict__ block_prefix, const __grid_constant__ RowTensors T,
                 const __grid_constant__ RowDsts D, int row_words)
{
    __shared__ uint32_t s_warp_cnt[RD_TILE / 32][RD_MAX_WS];
    __shared__ long long s_row[RD_TILE];     // exchange row of each row of the CTA (-1: dropped)
    __shared__ int s_dst[RD_TILE];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < (RD_TILE / 32) * RD_MAX_WS; k += RD_TILE) (&s_warp_cnt[0][0])[k] = 0;
    __syncthreads();
    const long long row0 = (long long)blockIdx.x * RD_TILE;
    const long long i = row0 + threadIdx.x;
    int d = -1;
    if (i < n) {
        d = destination[i];
        if (d < 0 || d >= ws) d = -1;
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    const uint32_t before = __popc(peers & ((1u << lane) - 1u));
    if (d >= 0 && before == 0) s_warp_cnt[warp][d] = __popc(peers);
    __syncthreads();
    long long row = -1;
    if (d >= 0) {
        uint32_t in_block = before;
        for (int w = 0; w < warp; w++) in_block += s_warp_cnt[w][d];
        row = D.first_row[d] + block_prefix[(size_t)d * nblocks + blockIdx.x] + in_block;
    }
    s_row[threadIdx.x] = row;
    s_dst[threadIdx.x] = d;
    __syncthreads();
    // cooperative copy: consecutive threads move consecutive words of a row (coalesced on both sides)
    const int rows_here = (int)min((long long)RD_TILE, n - row0);
    for (int t = 0; t < T.n; t++) {
        const int w = T.words[t];
        const uint32_t* src = reinterpret_cast<const uint32_t*>(T.ptr[t]) + row0 * w;
        const int total = rows_here * w;
        for (int e = threadIdx.x; e < total; e += RD_TILE) {
            const int r = e / w, c = e - r * w;
            const long long xr = s_row[r];
            if (xr >= 0) D.base[s_dst[r]][xr * row_words + T.offset[t] + c] = src[e];
        }
    }
}

// rows (n, row_words) -> tensor t gets columns [offset[t], offset[t] + words[t]) of every row
__global__ void __launch_bounds__(256)
rows_unpack_kernel(long long n, const uint32_t* __restrict__ rows, int row_words, const __grid_constant__ RowTensors T)
{
    const long long total = n * row_words;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const long long r = e / row_words;
        const int c = (int)(e - r * row_words);
        int t = 0;
        while (t + 1 < T.n && c >= T.offset[t + 1]) t++;
        reinterpret_cast<uint32_t*>(T.ptr[t])[r * T.words[t] + (c - T.offset[t])] = rows[e];
    }
}

// CTA j scans row j of the (ws, nblocks) table in place (exclusive) and writes the row total to counts[j].
__global__ void __launch_bounds__(1024)
rows_scan_kernel(int nblocks, uint32_t* __restrict__ block_counts, int32_t* __restrict__ counts)
{
    __shared__ uint32_t s_warp[32];
    __shared__ uint32_t s_carry;
    uint32_t* row = block_counts + (size_t)blockIdx.x * nblocks;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int start = 0; start < nblocks; start += 1024) {
        const int i = start + threadIdx.x;
        const uint32_t v = i < nblocks ? row[i] : 0;
        uint32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const uint32_t w = s_warp[lane];
            uint32_t wi = w;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t o = __shfl_up_sync(0xffffffffu, wi, d);
                if (lane >= d) wi += o;
            }
            s_warp[lane] = wi - w;
        }
        __syncthreads();
        const uint32_t excl = s_carry + s_warp[warp] + incl - v;
        if (i < nblocks) row[i] = excl;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[blockIdx.x] = (int32_t)s_carry;
}

static int fill_tensors(RowTensors& T, int n_tensors, void* const* ptrs, const int32_t* words_per_row)
{
    if (n_tensors <= 0 || n_tensors > RD_MAX_TENSORS || !ptrs || !words_per_row) return CGX_EINVAL;
    T.n = n_tensors;
    T.offset[0] = 0;
    for (int t = 0; t < RD_MAX_TENSORS; t++) {
        if (t < n_tensors) {
            if (words_per_row[t] <= 0 || !ptrs[t] || (reinterpret_cast<uintptr_t>(ptrs[t]) & 3)) return CGX_EINVAL;
            T.words[t] = words_per_row[t];
            T.ptr[t] = ptrs[t];
            T.offset[t + 1] = T.offset[t] + words_per_row[t];
        } else {
            T.words[t] = 0;
            T.ptr[t] = nullptr;
            T.offset[t + 1] = T.offset[t];
        }
    }
    return CGX_OK;
}

}  // namespace cgx

using namespace cgx;

extern "C" size_t cgx_rows_workspace_bytes(int64_t n, int ws)
{
    const size_t nblocks = ((size_t)(n > 0 ? n : 1) + RD_TILE - 1) / RD_TILE;
    return (nblocks * (size_t)(ws > 0 ? ws : 1) * sizeof(uint32_t) + 255) / 256 * 256 + 256;
}

extern "C" int cgx_rows_dest_count(int64_t n, int ws, const int32_t* destination, int32_t* counts, void* workspace,
                                   size_t workspace_bytes, void* stream)
{
    if (n < 0 || ws <= 0 || ws > RD_MAX_WS || !counts) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(counts, 0, (ws + 1) * sizeof(int32_t), st);      // counts[ws] = bad-destination flag
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    if (n == 0) return CGX_OK;
    if (!destination || !workspace) return CGX_EINVAL;
    if (workspace_bytes < cgx_rows_workspace_bytes(n, ws)) return CGX_ENOMEM;
    const int nblocks = (int)((n + RD_TILE - 1) / RD_TILE);
    rows_dest_count_kernel<<<nblocks, RD_TILE, 0, st>>>(n, ws, nblocks, destination, (uint32_t*)workspace, counts + ws);
    rows_scan_kernel<<<ws, 1024, 0, st>>>(nblocks, (uint32_t*)workspace, counts);
    return check_launch(2);
}

extern "C" int cgx_rows_pack(int64_t n, int ws, const int32_t* destination, int n_tensors, void* const* tensors,
                             const int32_t* words_per_row, uint32_t* const* dst_base, const int64_t* dst_first_row,
                             const void* workspace, void* stream)
{
    if (n < 0 || ws <= 0 || ws > RD_MAX_WS) return CGX_EINVAL;
    if (n == 0) return CGX_OK;
    if (!destination || !dst_base || !dst_first_row || !workspace) return CGX_EINVAL;
    RowTensors T;
    const int rc = fill_tensors(T, n_tensors, tensors, words_per_row);
    if (rc != CGX_OK) return rc;
    RowDsts D;
    for (int j = 0; j < RD_MAX_WS; j++) {
        D.base[j] = j < ws ? dst_base[j] : nullptr;
        D.first_row[j] = j < ws ? (long long)dst_first_row[j] : 0;
        if (j < ws && (dst_first_row[j] < 0 || (reinterpret_cast<uintptr_t>(dst_base[j]) & 3))) return CGX_EINVAL;
    }
    const int nblocks = (int)((n + RD_TILE - 1) / RD_TILE);
    rows_pack_kernel<<<nblocks, RD_TILE, 0, (cudaStream_t)stream>>>(n, ws, nblocks, destination,
                                                                   (const uint32_t*)workspace, T, D, T.offset[T.n]);
    return check_launch();
}

extern "C" int cgx_rows_unpack(int64_t n, const uint32_t* rows, int n_tensors, void* const* tensors,
                               const int32_t* words_per_row, void* stream)
{
    if (n < 0) return CGX_EINVAL;
    if (n == 0) return CGX_OK;
    if (!rows) return CGX_EINVAL;
    RowTensors T;
    const int rc = fill_tensors(T, n_tensors, tensors, words_per_row);
    if (rc != CGX_OK) return rc;
    const long long total = n * (long long)T.offset[T.n];
    const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    rows_unpack_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(n, rows, T.offset[T.n], T);
    return check_launch();
}
