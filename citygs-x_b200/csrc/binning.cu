// Binning stages: per-Gaussian tile counting + prefix sum, (tile|depth) key emission, the stable LSD
// radix sort of the key/value pairs, tile ranges, and the distribution masks / packers that drive the
// Gaussian all-to-all.  All integer / byte work, HBM-bound.
//
// Prefix sum: three launches without any inter-CTA waiting (count + CTA partial sums, one-CTA scan of
// the partial sums, emit with a CTA-local rescan).  The radix sort keeps digit histograms on chip
// (per-warp shared-memory counters filled with match.any ballots), again without inter-CTA spin waits:
// per pass a histogram kernel, a 256-CTA digit-row scan and a scatter kernel that stages each CTA's
// keys in shared memory so that every digit run leaves as a contiguous burst.
#include "cgx_common.cuh"

namespace cgx {

// ------------------------------------------------------------------------------------------------ scan
constexpr int SCAN_ITEMS = 4;                              // Gaussians per thread in count / emit
constexpr int SCAN_TILE = CGX_BLOCK_SIZE * SCAN_ITEMS;     // Gaussians per CTA

// The local-tile mask as a band of whole tile rows [row0, row1), when it is one (it always is for the workload
// division's row bands and for a single GPU): valid = 1 lets the counting and emission kernels replace one mask
// lookup per tile by two comparisons per splat.  Any other mask (valid = 0) goes through the lookups.
struct MaskBand {
    int valid, row0, row1, pad;
};

__global__ void __launch_bounds__(1024)
analyse_mask_kernel(int gx, int gy, const uint8_t* __restrict__ local, MaskBand* __restrict__ band)
{
    __shared__ int s_partial, s_first, s_last, s_full;
    if (threadIdx.x == 0) {
        s_partial = 0;
        s_first = gy;
        s_last = -1;
        s_full = 0;
    }
    __syncthreads();
    for (int y = threadIdx.x; y < gy; y += blockDim.x) {
        int set = 0;
        for (int x = 0; x < gx; x++) set += local[y * gx + x] ? 1 : 0;
        if (set == gx) {
            atomicMin(&s_first, y);
            atomicMax(&s_last, y);
            atomicAdd(&s_full, 1);
        } else if (set != 0) {
            atomicExch(&s_partial, 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        MaskBand b;
        b.pad = 0;
        if (s_full == 0 && !s_partial) {
            b.valid = 1; b.row0 = 0; b.row1 = 0;                    // nothing is local
        } else {
            b.valid = (!s_partial && s_full == s_last - s_first + 1) ? 1 : 0;
            b.row0 = s_first;
            b.row1 = s_last + 1;
        }
        *band = b;
    }
}

__device__ __forceinline__ uint32_t count_local_tiles(const float2 xy, int radius, const uint8_t* __restrict__ local,
                                                      int gx, int gy, const MaskBand band)
{
    uint32_t cnt = 0;
    if (radius > 0) {
        uint2 rect_min, rect_max;
        get_rect(xy, radius, rect_min, rect_max, gx, gy);
        if (band.valid) {
            const int rows = min((int)rect_max.y, band.row1) - max((int)rect_min.y, band.row0);
            const int cols = (int)rect_max.x - (int)rect_min.x;
            cnt = (rows > 0 && cols > 0) ? (uint32_t)(rows * cols) : 0u;
        } else {
            for (int y = rect_min.y; y < rect_max.y; y++)
                for (int x = rect_min.x; x < rect_max.x; x++)
                    if (local[y * gx + x]) cnt++;
        }
    }
    return cnt;
}

__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t v)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t n = __shfl_up_sync(0xffffffffu, v, d);
        if ((threadIdx.x & 31) >= d) v += n;
    }
    return v;
}

// Exclusive prefix of `v` over the CTA (256 threads); returns the CTA total through `total`.
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t* s_warp /*[8]*/, uint32_t& total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t incl = warp_incl_scan(v);
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t wbase = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < CGX_BLOCK_SIZE / 32; w++) {
        uint32_t s = s_warp[w];
        if (w < warp) wbase += s;
        tot += s;
    }
    total = tot;
    __syncthreads();
    return wbase + incl - v;
}

__global__ void __launch_bounds__(CGX_BLOCK_SIZE)
tile_count_kernel(int P, int gx, int gy, const int* __restrict__ radii, const float2* __restrict__ means2D,
                  const uint8_t* __restrict__ local, uint32_t* __restrict__ tiles_touched,
                  uint32_t* __restrict__ block_sums, const MaskBand* __restrict__ band_ptr,
                  const float* __restrict__ depths, uint32_t* __restrict__ depth_range, const int vec_ok)
{
    __shared__ uint32_t s_warp[8];
    const MaskBand band = *band_ptr;
    const int base = blockIdx.x * SCAN_TILE;
    uint32_t sum = 0;
    uint32_t dmin = 0xffffffffu, dmax = 0u;     // bit patterns of the depths of the splats that emit keys
    // a thread owns SCAN_ITEMS consecutive Gaussians: its loads and its store are 128-bit wide
    const int idx0 = base + threadIdx.x * SCAN_ITEMS;
    if (idx0 + SCAN_ITEMS <= P && vec_ok) {
        const float4 m01 = *reinterpret_cast<const float4*>(means2D + idx0);
        const float4 m23 = *reinterpret_cast<const float4*>(means2D + idx0 + 2);
        const int4 rad = *reinterpret_cast<const int4*>(radii + idx0);
        uint4 c;
        c.x = count_local_tiles(make_float2(m01.x, m01.y), rad.x, local, gx, gy, band);
        c.y = count_local_tiles(make_float2(m01.z, m01.w), rad.y, local, gx, gy, band);
        c.z = count_local_tiles(make_float2(m23.x, m23.y), rad.z, local, gx, gy, band);
        c.w = count_local_tiles(make_float2(m23.z, m23.w), rad.w, local, gx, gy, band);
        *reinterpret_cast<uint4*>(tiles_touched + idx0) = c;
        sum = c.x + c.y + c.z + c.w;
        if (depths && sum) {
            const float4 d = *reinterpret_cast<const float4*>(depths + idx0);
            const uint32_t cs[4] = {c.x, c.y, c.z, c.w};
            const float ds[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int k = 0; k < SCAN_ITEMS; k++)
                if (cs[k]) {
                    const uint32_t b = __float_as_uint(ds[k]);
                    dmin = min(dmin, b);
                    dmax = max(dmax, b);
                }
        }
    } else {
        for (int k = 0; k < SCAN_ITEMS; k++) {
            const int idx = idx0 + k;
            if (idx < P) {
                const uint32_t c = count_local_tiles(means2D[idx], radii[idx], local, gx, gy, band);
                tiles_touched[idx] = c;
                sum += c;
                if (depths && c) {
                    const uint32_t b = __float_as_uint(depths[idx]);
                    dmin = min(dmin, b);
                    dmax = max(dmax, b);
                }
            }
        }
    }
    uint32_t total;
    block_excl_scan(sum, s_warp, total);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
    if (depths) {
        // per-CTA range, left beside the CTA's sum: the one-CTA scan kernel reduces them (no atomics on one word)
        __shared__ uint32_t s_min[8], s_max[8];
        dmin = __reduce_min_sync(0xffffffffu, dmin);
        dmax = __reduce_max_sync(0xffffffffu, dmax);
        if ((threadIdx.x & 31) == 0) {
            s_min[threadIdx.x >> 5] = dmin;
            s_max[threadIdx.x >> 5] = dmax;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; w++) {
                dmin = min(dmin, s_min[w]);
                dmax = max(dmax, s_max[w]);
            }
            depth_range[2 * blockIdx.x] = dmin;
            depth_range[2 * blockIdx.x + 1] = dmax;
        }
    }
}


// In-place exclusive scan of row[0..n) by one 1024-thread CTA; returns the row total (valid on every thread).
__device__ __forceinline__ uint32_t scan_row_inplace(uint32_t* __restrict__ row, int n)
{
    __shared__ uint32_t s_warp[32];
    __shared__ uint32_t s_carry;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int start = 0; start < n; start += 1024) {
        const int i = start + threadIdx.x;
        const uint32_t v = i < n ? row[i] : 0;
        uint32_t incl = warp_incl_scan(v);
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            uint32_t w = s_warp[lane];
            uint32_t wi = warp_incl_scan(w);
            s_warp[lane] = wi - w;
        }
        __syncthreads();
        const uint32_t excl = s_carry + s_warp[warp] + incl - v;
        if (i < n) row[i] = excl;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = excl + v;
        __syncthreads();
    }
    return s_carry;
}

// One CTA: in-place exclusive scan of the CTA partial sums; writes the grand total.
// block_ranges (optional): per-CTA (min, max) depth bit patterns -> total_out[1], total_out[2].
__global__ void __launch_bounds__(1024)
scan_partials_kernel(int n, uint32_t* __restrict__ sums, uint32_t* __restrict__ total_out,
                     const uint32_t* __restrict__ block_ranges)
{
    const uint32_t total = scan_row_inplace(sums, n);
    if (threadIdx.x == 0) total_out[0] = total;
    if (block_ranges) {
        __shared__ uint32_t s_min[32], s_max[32];
        uint32_t lo = 0xffffffffu, hi = 0u;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            lo = min(lo, block_ranges[2 * i]);
            hi = max(hi, block_ranges[2 * i + 1]);
        }
        lo = __reduce_min_sync(0xffffffffu, lo);
        hi = __reduce_max_sync(0xffffffffu, hi);
        if ((threadIdx.x & 31) == 0) {
            s_min[threadIdx.x >> 5] = lo;
            s_max[threadIdx.x >> 5] = hi;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 32; w++) {
                lo = min(lo, s_min[w]);
                hi = max(hi, s_max[w]);
            }
            total_out[1] = lo;
            total_out[2] = hi;
        }
    }
}

__global__ void __launch_bounds__(CGX_BLOCK_SIZE)
emit_keys_kernel(int P, int gx, int gy, const int* __restrict__ radii, const float2* __restrict__ means2D,
                 const float* __restrict__ depths, const uint32_t* __restrict__ tiles_touched,
                 const uint8_t* __restrict__ local, const uint32_t* __restrict__ block_prefix,
                 uint32_t* __restrict__ point_offsets, uint64_t* __restrict__ keys, uint32_t* __restrict__ values,
                 uint32_t capacity, const MaskBand* __restrict__ band_ptr, const int vec_ok)
{
    __shared__ uint32_t s_warp[8];
    const MaskBand band = *band_ptr;
    const int base = blockIdx.x * SCAN_TILE;
    // a thread owns SCAN_ITEMS consecutive Gaussians (as in the counting kernel): one CTA-wide scan of the threads'
    // sums gives every thread its first output position, the counts inside the thread give the rest
    const int idx0 = base + threadIdx.x * SCAN_ITEMS;
    const bool vec = idx0 + SCAN_ITEMS <= P && vec_ok;
    uint32_t c[SCAN_ITEMS];
    if (vec) {
        const uint4 t = *reinterpret_cast<const uint4*>(tiles_touched + idx0);
        c[0] = t.x; c[1] = t.y; c[2] = t.z; c[3] = t.w;
    } else {
#pragma unroll
        for (int k = 0; k < SCAN_ITEMS; k++) c[k] = idx0 + k < P ? tiles_touched[idx0 + k] : 0;
    }
    uint32_t total;
    uint32_t off = block_prefix[blockIdx.x] + block_excl_scan(c[0] + c[1] + c[2] + c[3], s_warp, total);
    if (vec) {
        *reinterpret_cast<uint4*>(point_offsets + idx0) =
            make_uint4(off + c[0], off + c[0] + c[1], off + c[0] + c[1] + c[2], off + c[0] + c[1] + c[2] + c[3]);
    } else {
        uint32_t run = off;
        for (int k = 0; k < SCAN_ITEMS; k++)
            if (idx0 + k < P) {
                run += c[k];
                point_offsets[idx0 + k] = run;
            }
    }
    if (c[0] + c[1] + c[2] + c[3] == 0) return;
#pragma unroll 1
    for (int k = 0; k < SCAN_ITEMS; k++) {
        const int idx = idx0 + k;
        if (c[k] > 0) {
            const float2 xy = means2D[idx];
            uint2 rect_min, rect_max;
            get_rect(xy, radii[idx], rect_min, rect_max, gx, gy);
            const uint64_t dbits = (uint64_t)__float_as_uint(depths[idx]);
            // a band of whole rows: its rows of the rectangle are local, the others are not
            const int y0 = band.valid ? max((int)rect_min.y, band.row0) : (int)rect_min.y;
            const int y1 = band.valid ? min((int)rect_max.y, band.row1) : (int)rect_max.y;
            for (int y = y0; y < y1; y++)
                for (int x = rect_min.x; x < rect_max.x; x++)
                    if (band.valid || local[y * gx + x]) {
                        if (off < capacity) {
                            uint64_t key = y * gx + x;
                            key <<= 32;
                            key |= dbits;
                            keys[off] = key;
                            values[off] = idx;
                        }
                        off++;
                    }
        }
    }
}

// ------------------------------------------------------------------------------------------------ sort
constexpr int SORT_THREADS = 256;
#ifndef CGX_SORT_ITEMS
#define CGX_SORT_ITEMS 8
#endif
constexpr int SORT_ITEMS = CGX_SORT_ITEMS;
constexpr int SORT_TILE = SORT_THREADS * SORT_ITEMS;  // 2048 pairs per CTA (measured best of 1024 / 2048 / 4096)
constexpr int RADIX_BITS = 8;
constexpr int RADIX = 1 << RADIX_BITS;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int SORT_SMEM = SORT_TILE * (sizeof(uint64_t) + sizeof(uint32_t));

// Digit of a key.  Keys are (tile << 32) | depth bits.  When the caller knows that bits [low_bits, 32) of the low
// word are the same in every key (depths of one view share their sign, most of their exponent ...), those bits
// cannot change the order and are squeezed out: the sort then runs over low_bits + tile bits, often one pass fewer.
// Which bits of the two key words make up the digit of a pass is worked out on the host once per pass:
//   digit = ((lo >> s_lo) & m_lo) | (((hi >> r_hi) << l_hi) & m_hi)
struct DigitSpec {
    uint32_t s_lo, m_lo, r_hi, l_hi, m_hi;
};

__host__ __device__ __forceinline__ DigitSpec digit_spec(int shift, uint32_t mask, int low_bits)
{
    DigitSpec d;
    if (shift >= low_bits) {                 // the whole digit comes from the high word
        d = {0u, 0u, (uint32_t)(shift - low_bits), 0u, mask};
    } else {
        const int from_lo = low_bits - shift;            // bits the low word still has at this shift
        const uint32_t m_lo = from_lo >= 32 ? 0xffffffffu : ((1u << from_lo) - 1u);
        d = {(uint32_t)shift, m_lo & mask, 0u, (uint32_t)(from_lo >= 32 ? 0 : from_lo), from_lo >= 32 ? 0u : (mask & ~m_lo)};
    }
    return d;
}

__device__ __forceinline__ uint32_t sort_digit(uint64_t k, const DigitSpec d)
{
    const uint32_t lo = (uint32_t)k, hi = (uint32_t)(k >> 32);
    return ((lo >> d.s_lo) & d.m_lo) | (((hi >> d.r_hi) << d.l_hi) & d.m_hi);
}

// table layout: counts[digit * nblocks + block]
__global__ void __launch_bounds__(SORT_THREADS)
sort_hist_kernel(int64_t n, int nblocks, const DigitSpec dg, const uint64_t* __restrict__ keys,
                 uint32_t* __restrict__ table)
{
    __shared__ uint32_t s_hist[RADIX];
    for (int i = threadIdx.x; i < RADIX; i += SORT_THREADS) s_hist[i] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * SORT_TILE;
#pragma unroll 4
    for (int k = 0; k < SORT_ITEMS; k++) {
        const int64_t i = base + k * SORT_THREADS + threadIdx.x;
        if (i < n) {
            const uint32_t d = sort_digit(keys[i], dg);
            atomicAdd(&s_hist[d], 1u);
        }
    }
    __syncthreads();
    for (int d = threadIdx.x; d < RADIX; d += SORT_THREADS) table[(size_t)d * nblocks + blockIdx.x] = s_hist[d];
}

// CTA d scans row d of the table (exclusive, in place) and leaves the digit total in totals[d].
__global__ void __launch_bounds__(1024)
sort_scan_rows_kernel(int nblocks, uint32_t* __restrict__ table, uint32_t* __restrict__ totals)
{
    const uint32_t total = scan_row_inplace(table + (size_t)blockIdx.x * nblocks, nblocks);
    if (threadIdx.x == 0) totals[blockIdx.x] = total;
}

// Stable scatter of one tile of SORT_TILE pairs.  Warp w owns SORT_ITEMS consecutive "rounds" of its contiguous
// chunk of 32*SORT_ITEMS pairs: in round r the warp looks at pairs [chunk + 32 r, chunk + 32 r + 32), so
// (warp, round, lane) order is input order and ranks computed from match.any ballots are stable.
__global__ void __launch_bounds__(SORT_THREADS)
sort_scatter_kernel(int64_t n, int nblocks, const DigitSpec dg, const uint64_t* __restrict__ keys_in,
                    const uint32_t* __restrict__ vals_in, uint64_t* __restrict__ keys_out,
                    uint32_t* __restrict__ vals_out, const uint32_t* __restrict__ table,
                    const uint32_t* __restrict__ totals)
{
    __shared__ uint32_t s_warp_hist[SORT_WARPS][RADIX];  // per-warp digit counters, then exclusive warp offsets
    __shared__ uint32_t s_digit_start[RADIX];            // start of each digit run inside the CTA's staged tile
    __shared__ uint32_t s_global_base[RADIX];            // global position of the CTA's first pair of each digit
    extern __shared__ __align__(16) unsigned char s_dyn[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_dyn);
    uint32_t* s_vals = reinterpret_cast<uint32_t*>(s_dyn + SORT_TILE * sizeof(uint64_t));

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < SORT_WARPS * RADIX; i += SORT_THREADS) (&s_warp_hist[0][0])[i] = 0;

    // global base of every digit: sum of the totals of smaller digits + this CTA's offset inside its digit row
    {
        const int d = threadIdx.x;  // SORT_THREADS == RADIX
        uint32_t t = totals[d];
        uint32_t incl = warp_incl_scan(t);
        __shared__ uint32_t s_w[SORT_WARPS];
        if (lane == 31) s_w[warp] = incl;
        __syncthreads();
        uint32_t wb = 0;
#pragma unroll
        for (int w = 0; w < SORT_WARPS; w++)
            if (w < warp) wb += s_w[w];
        s_global_base[d] = wb + incl - t + table[(size_t)d * nblocks + blockIdx.x];
    }
    __syncthreads();

    const int64_t tile_base = (int64_t)blockIdx.x * SORT_TILE;
    const int64_t chunk = tile_base + (int64_t)warp * (32 * SORT_ITEMS);
    uint64_t key[SORT_ITEMS];
    uint32_t val[SORT_ITEMS];
    uint32_t rank[SORT_ITEMS];  // rank of the pair among same-digit pairs of this warp

#pragma unroll
    for (int r = 0; r < SORT_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        const bool valid = i < n;
        key[r] = valid ? keys_in[i] : ~0ull;
        val[r] = valid ? vals_in[i] : 0u;
    }
#pragma unroll
    for (int r = 0; r < SORT_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        const bool valid = i < n;
        // invalid tail lanes take a digit of their own (RADIX) so they never match a real digit
        const uint32_t d = valid ? sort_digit(key[r], dg) : (uint32_t)RADIX;
        const uint32_t peers = __match_any_sync(0xffffffffu, d);
        const uint32_t before = __popc(peers & ((1u << lane) - 1u));
        uint32_t prev = 0;
        if (valid && before == 0) {  // first lane of its digit group updates the warp counter
            prev = s_warp_hist[warp][d];
            s_warp_hist[warp][d] = prev + __popc(peers);
        }
        prev = __shfl_sync(0xffffffffu, prev, __ffs(peers) - 1);
        rank[r] = prev + before;
        __syncwarp();
    }
    __syncthreads();

    // per digit: exclusive prefix over the warps, CTA total; then exclusive scan over digits
    {
        const int d = threadIdx.x;
        uint32_t run = 0;
#pragma unroll
        for (int w = 0; w < SORT_WARPS; w++) {
            uint32_t c = s_warp_hist[w][d];
            s_warp_hist[w][d] = run;
            run += c;
        }
        uint32_t incl = warp_incl_scan(run);
        __shared__ uint32_t s_w2[SORT_WARPS];
        if (lane == 31) s_w2[warp] = incl;
        __syncthreads();
        uint32_t wb = 0;
#pragma unroll
        for (int w = 0; w < SORT_WARPS; w++)
            if (w < warp) wb += s_w2[w];
        s_digit_start[d] = wb + incl - run;
    }
    __syncthreads();

    // stage the tile in digit order
#pragma unroll
    for (int r = 0; r < SORT_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        if (i < n) {
            const uint32_t d = sort_digit(key[r], dg);
            const uint32_t pos = s_digit_start[d] + s_warp_hist[warp][d] + rank[r];
            s_keys[pos] = key[r];
            s_vals[pos] = val[r];
        }
    }
    __syncthreads();

    const int valid_n = (int)min((int64_t)SORT_TILE, n - tile_base);
    for (int p = threadIdx.x; p < valid_n; p += SORT_THREADS) {
        const uint64_t k = s_keys[p];
        const uint32_t d = sort_digit(k, dg);
        const size_t dst = (size_t)s_global_base[d] + (p - s_digit_start[d]);
        keys_out[dst] = k;
        vals_out[dst] = s_vals[p];
    }
}

// Scatter without staging: ranks are computed as above, but the keys are not kept in registers and the pairs are
// written straight to their final positions.  Few registers (8 CTAs per SM); the scattered 8- and 4-byte stores are
// merged in L2, which is the right trade while both ping-pong buffers fit in L2 (n * 24 bytes well below 126 MB).
__global__ void __launch_bounds__(SORT_THREADS, 6)
sort_scatter_direct_kernel(int64_t n, int nblocks, const DigitSpec dg, const uint64_t* __restrict__ keys_in,
                           const uint32_t* __restrict__ vals_in, uint64_t* __restrict__ keys_out,
                           uint32_t* __restrict__ vals_out, const uint32_t* __restrict__ table,
                           const uint32_t* __restrict__ totals)
{
    __shared__ uint32_t s_warp_hist[SORT_WARPS][RADIX];  // per-warp digit counters, then global position of the
                                                         // warp's first pair of each digit
    __shared__ uint32_t s_w[SORT_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < SORT_WARPS * RADIX; i += SORT_THREADS) (&s_warp_hist[0][0])[i] = 0;
    __syncthreads();

    const int64_t tile_base = (int64_t)blockIdx.x * SORT_TILE;
    const int64_t chunk = tile_base + (int64_t)warp * (32 * SORT_ITEMS);
    uint16_t rank[SORT_ITEMS];
#pragma unroll
    for (int r = 0; r < SORT_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        const bool valid = i < n;
        const uint32_t d = valid ? sort_digit(keys_in[i], dg) : (uint32_t)RADIX;
        const uint32_t peers = __match_any_sync(0xffffffffu, d);
        const uint32_t before = __popc(peers & ((1u << lane) - 1u));
        uint32_t prev = 0;
        if (valid && before == 0) {
            prev = s_warp_hist[warp][d];
            s_warp_hist[warp][d] = prev + __popc(peers);
        }
        prev = __shfl_sync(0xffffffffu, prev, __ffs(peers) - 1);
        rank[r] = (uint16_t)(prev + before);
        __syncwarp();
    }
    __syncthreads();
    {
        // digit d: global base = totals of smaller digits + this CTA's offset in the digit row; then per warp
        const int d = threadIdx.x;
        const uint32_t t = totals[d];
        const uint32_t incl = warp_incl_scan(t);
        if (lane == 31) s_w[warp] = incl;
        __syncthreads();
        uint32_t wb = 0;
#pragma unroll
        for (int w = 0; w < SORT_WARPS; w++)
            if (w < warp) wb += s_w[w];
        uint32_t run = wb + incl - t + table[(size_t)d * nblocks + blockIdx.x];
#pragma unroll
        for (int w = 0; w < SORT_WARPS; w++) {
            const uint32_t c = s_warp_hist[w][d];
            s_warp_hist[w][d] = run;
            run += c;
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < SORT_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        if (i < n) {
            const uint64_t k = keys_in[i];
            const uint32_t d = sort_digit(k, dg);
            const size_t dst = (size_t)s_warp_hist[warp][d] + rank[r];
            keys_out[dst] = k;
            vals_out[dst] = vals_in[i];
        }
    }
}

// ------------------------------------------------------------------------------------------------ one-sweep sort
// One read of the keys builds the digit histograms of ALL passes (global totals only).  Each pass is then ONE
// kernel: a CTA takes the next tile (a ticket, so every tile it will ever wait for is already running), ranks its
// pairs by digit on chip (match.any ballots, per-warp counters), publishes its per-digit counts, finds the number
// of same-digit pairs in earlier tiles by decoupled look-back over the published counts, and scatters.  Per pass
// the pairs are read once and written once; nothing else touches HBM but 1 KB of counts per tile.
// The look-back is the only place a CTA waits for another one; the wait is bounded (clock64) and sets the device
// status word when it gives up.
constexpr int OS_THREADS = 256;
#ifndef CGX_OS_ITEMS
#define CGX_OS_ITEMS 16
#endif
#ifndef CGX_OS_MIN_CTAS
#define CGX_OS_MIN_CTAS 2
#endif
constexpr int OS_ITEMS = CGX_OS_ITEMS;
constexpr int OS_TILE = OS_THREADS * OS_ITEMS;
constexpr int OS_WARPS = OS_THREADS / 32;
constexpr int OS_MAX_PASSES = 8;
constexpr uint32_t OS_FLAG_AGG = 1u << 30;      // value = pairs of this digit in this tile
constexpr uint32_t OS_FLAG_PREFIX = 2u << 30;   // value = pairs of this digit in this tile and all earlier ones
constexpr uint32_t OS_VALUE_MASK = (1u << 30) - 1u;
constexpr unsigned long long OS_WAIT_LIMIT_CYCLES = 1ull << 28;   // ~0.14 s at B200 clocks

__device__ int g_sort_status = 0;   // CGX_ETIMEDOUT when a look-back wait gave up

__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu(uint32_t* p, uint32_t v)
{
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ghist[pass * RADIX + digit] += number of keys with that digit in that pass.
__global__ void __launch_bounds__(OS_THREADS)
os_hist_kernel(int64_t n, int passes, int end_bit, int low_bits, const uint64_t* __restrict__ keys,
               uint32_t* __restrict__ ghist)
{
    __shared__ uint32_t s_hist[OS_MAX_PASSES * RADIX];
    for (int i = threadIdx.x; i < passes * RADIX; i += OS_THREADS) s_hist[i] = 0;
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * OS_THREADS;
    const int lane = threadIdx.x & 31;
    // i0 is the same for all lanes of a warp, so every lane takes part in every vote
    for (int64_t i0 = (int64_t)blockIdx.x * OS_THREADS + (threadIdx.x & ~31); i0 < n; i0 += stride) {
        const bool valid = i0 + lane < n;
        const uint64_t k = valid ? keys[i0 + lane] : 0ull;
        for (int p = 0; p < passes; p++) {
            const int shift = p * RADIX_BITS;
            const int bits = min(RADIX_BITS, end_bit - shift);
            const uint32_t d = valid ? sort_digit(k, digit_spec(shift, (1u << bits) - 1u, low_bits)) : (uint32_t)RADIX;
            // lanes of a warp often share a digit in the high passes (few tiles, few exponents): one add per group
            const uint32_t peers = __match_any_sync(0xffffffffu, d);
            if (valid && lane == __ffs(peers) - 1) atomicAdd(&s_hist[p * RADIX + d], (uint32_t)__popc(peers));
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < passes * RADIX; i += OS_THREADS) {
        const uint32_t c = s_hist[i];
        if (c) atomicAdd(&ghist[i], c);
    }
}

__global__ void __launch_bounds__(OS_THREADS, CGX_OS_MIN_CTAS)
os_pass_kernel(int64_t n, const DigitSpec dg, const uint64_t* __restrict__ keys_in,
               const uint32_t* __restrict__ vals_in, uint64_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
               const uint32_t* __restrict__ ghist, uint32_t* __restrict__ ticket, uint32_t* __restrict__ status,
               unsigned long long wait_limit)
{
    __shared__ uint32_t s_warp_hist[OS_WARPS][RADIX];  // per-warp digit counters, then exclusive offsets over warps
    __shared__ uint32_t s_base[RADIX];                 // global position of the tile's first pair of each digit
    __shared__ uint32_t s_w[OS_WARPS];
    __shared__ uint32_t s_tile;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1u);
    for (int i = threadIdx.x; i < OS_WARPS * RADIX; i += OS_THREADS) (&s_warp_hist[0][0])[i] = 0;
    __syncthreads();
    const uint32_t tile = s_tile;
    const int64_t tile_base = (int64_t)tile * OS_TILE;
    if (tile_base >= n) return;                        // uniform over the CTA (cannot happen with an exact grid)
    const int64_t chunk = tile_base + (int64_t)warp * (32 * OS_ITEMS);

    uint64_t key[OS_ITEMS];
    uint16_t rank[OS_ITEMS];
#pragma unroll
    for (int r = 0; r < OS_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        key[r] = i < n ? keys_in[i] : ~0ull;
    }
#pragma unroll
    for (int r = 0; r < OS_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        const bool valid = i < n;
        // invalid tail lanes take a digit of their own (RADIX) so they never match a real digit
        const uint32_t d = valid ? sort_digit(key[r], dg) : (uint32_t)RADIX;
        const uint32_t peers = __match_any_sync(0xffffffffu, d);
        const uint32_t before = __popc(peers & ((1u << lane) - 1u));
        uint32_t prev = 0;
        if (valid && before == 0) {  // first lane of its digit group updates the warp counter
            prev = s_warp_hist[warp][d];
            s_warp_hist[warp][d] = prev + __popc(peers);
        }
        prev = __shfl_sync(0xffffffffu, prev, __ffs(peers) - 1);
        rank[r] = (uint16_t)(prev + before);
        __syncwarp();
    }
    __syncthreads();

    bool failed = false;
    {
        const int d = threadIdx.x;  // OS_THREADS == RADIX
        uint32_t cnt = 0;
#pragma unroll
        for (int w = 0; w < OS_WARPS; w++) {
            const uint32_t c = s_warp_hist[w][d];
            s_warp_hist[w][d] = cnt;
            cnt += c;
        }
        uint32_t* my_status = status + (size_t)tile * RADIX + d;
        st_relaxed_gpu(my_status, (tile == 0 ? OS_FLAG_PREFIX : OS_FLAG_AGG) | cnt);
        // first pair of digit d in the whole array: totals of the smaller digits
        const uint32_t t = ghist[d];
        const uint32_t incl = warp_incl_scan(t);
        if (lane == 31) s_w[warp] = incl;
        __syncthreads();
        uint32_t digit_base = incl - t;
#pragma unroll
        for (int w = 0; w < OS_WARPS; w++)
            if (w < warp) digit_base += s_w[w];
        // pairs of digit d in earlier tiles: walk back until a tile that already knows its inclusive prefix
        uint32_t excl = 0;
        if (tile > 0) {
            const long long t0 = clock64();
            for (int64_t b = (int64_t)tile - 1; b >= 0; b--) {
                const uint32_t* p = status + (size_t)b * RADIX + d;
                uint32_t v = ld_relaxed_gpu(p);
                while ((v >> 30) == 0) {
                    if ((unsigned long long)(clock64() - t0) > wait_limit) {
                        failed = true;
                        break;
                    }
                    v = ld_relaxed_gpu(p);
                }
                if (failed) break;
                excl += v & OS_VALUE_MASK;
                if (v & OS_FLAG_PREFIX) break;
            }
            if (!failed) st_relaxed_gpu(my_status, OS_FLAG_PREFIX | (excl + cnt));
        }
        s_base[d] = digit_base + excl;
    }
    if (__syncthreads_or(failed)) {
        if (threadIdx.x == 0) atomicExch(&g_sort_status, CGX_ETIMEDOUT);
        return;      // nothing is scattered: the output of this tile is undefined and the status word says so
    }
#pragma unroll
    for (int r = 0; r < OS_ITEMS; r++) {
        const int64_t i = chunk + r * 32 + lane;
        if (i < n) {
            const uint32_t d = sort_digit(key[r], dg);
            const size_t dst = (size_t)s_base[d] + s_warp_hist[warp][d] + rank[r];
            keys_out[dst] = key[r];
            vals_out[dst] = vals_in[i];
        }
    }
}

__global__ void __launch_bounds__(256)
tile_ranges_kernel(int64_t L, uint32_t T, const uint64_t* __restrict__ keys, uint2* __restrict__ ranges)
{
    // A tile id beyond the grid can only come from a key nobody emitted (a caller that passed a pair count larger
    // than the emitted one): such a key never writes, so nothing outside `ranges` is touched.
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= L) return;
    const uint32_t currtile = (uint32_t)(keys[idx] >> 32);
    const bool cur_ok = currtile < T;
    if (idx == 0) {
        if (cur_ok) ranges[currtile].x = 0;
    } else {
        const uint32_t prevtile = (uint32_t)(keys[idx - 1] >> 32);
        if (currtile != prevtile) {
            if (prevtile < T) ranges[prevtile].y = (uint32_t)idx;
            if (cur_ok) ranges[currtile].x = (uint32_t)idx;
        }
    }
    if (idx == L - 1 && cur_ok) ranges[currtile].y = (uint32_t)L;
}

// ------------------------------------------------------------------------------------------------ distribution
__device__ __forceinline__ bool touches_band(int tmin, int tmax, int tile_l, int tile_r, int gx, bool avoid)
{
    if (avoid) {
        tile_l -= gx + 1;
        tile_r += gx + 1;
    }
    return !(tmax < tile_l || tmin >= tile_r);
}

__global__ void __launch_bounds__(256)
local2j_mask_kernel(int P, int gx, int gy, int ws, const float2* __restrict__ means2D, const int* __restrict__ radii,
                    const int* __restrict__ bounds, bool avoid, uint8_t* __restrict__ mask)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P) return;
    uint2 rect_min, rect_max;
    get_rect(means2D[i], radii[i], rect_min, rect_max, gx, gy);
    const int tmin = rect_min.y * gx + rect_min.x;
    const int tmax = ((int)rect_max.y - 1) * gx + (int)rect_max.x - 1;
    const bool any = !(tmax < tmin);
    for (int rk = 0; rk < ws; rk++)
        mask[(size_t)i * ws + rk] = any && touches_band(tmin, tmax, bounds[rk], bounds[rk + 1], gx, avoid);
}

constexpr int MAX_WS = 32;
#ifndef CGX_PACK_TILE
#define CGX_PACK_TILE 256
#endif
constexpr int PACK_TILE = CGX_PACK_TILE;  // rows per CTA (and threads per CTA) of the exchange's count / pack kernels

// counts[j] (global) and per-CTA counts block_counts[j * nblocks + b]
__global__ void __launch_bounds__(PACK_TILE)
local2j_count_kernel(int P, int gx, int gy, int ws, int nblocks, const float2* __restrict__ means2D,
                     const int* __restrict__ radii, const int* __restrict__ bounds, bool avoid,
                     uint32_t* __restrict__ block_counts)
{
    __shared__ uint32_t s_cnt[MAX_WS];
    if (threadIdx.x < MAX_WS) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    const int i = blockIdx.x * PACK_TILE + threadIdx.x;
    uint32_t bits = 0;
    if (i < P) {
        uint2 rect_min, rect_max;
        get_rect(means2D[i], radii[i], rect_min, rect_max, gx, gy);
        const int tmin = rect_min.y * gx + rect_min.x;
        const int tmax = ((int)rect_max.y - 1) * gx + (int)rect_max.x - 1;
        if (!(tmax < tmin))
            for (int rk = 0; rk < ws; rk++)
                if (touches_band(tmin, tmax, bounds[rk], bounds[rk + 1], gx, avoid)) bits |= 1u << rk;
    }
    for (int rk = 0; rk < ws; rk++) {
        const uint32_t b = __ballot_sync(0xffffffffu, (bits >> rk) & 1u);
        if ((threadIdx.x & 31) == 0 && b) atomicAdd(&s_cnt[rk], __popc(b));
    }
    __syncthreads();
    if (threadIdx.x < ws) block_counts[(size_t)threadIdx.x * nblocks + blockIdx.x] = s_cnt[threadIdx.x];
}

// CTA j scans row j of block_counts in place (exclusive) and writes counts[j].
__global__ void __launch_bounds__(1024)
local2j_scan_kernel(int nblocks, uint32_t* __restrict__ block_counts, int32_t* __restrict__ counts)
{
    const uint32_t total = scan_row_inplace(block_counts + (size_t)blockIdx.x * nblocks, nblocks);
    if (threadIdx.x == 0) counts[blockIdx.x] = (int32_t)total;
}

// The counting stage of every camera of a batch in two launches (blockIdx.y = camera).
constexpr int MAX_COUNT_CAMS = 16;
struct CountCamera {
    const float2* means2D;
    const int* radii;
    const int* bounds;
    uint32_t* block_counts;
    int32_t* counts;
    int P, gx, gy, ws, nblocks, avoid;
};
struct CountBatch {
    CountCamera cam[MAX_COUNT_CAMS];
};

__global__ void __launch_bounds__(PACK_TILE)
local2j_count_batched_kernel(const __grid_constant__ CountBatch b)
{
    const CountCamera& c = b.cam[blockIdx.y];
    if ((int)blockIdx.x >= c.nblocks) return;          // uniform over the CTA
    __shared__ uint32_t s_cnt[MAX_WS];
    if (threadIdx.x < MAX_WS) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    const int i = blockIdx.x * PACK_TILE + threadIdx.x;
    uint32_t bits = 0;
    if (i < c.P) {
        uint2 rect_min, rect_max;
        get_rect(c.means2D[i], c.radii[i], rect_min, rect_max, c.gx, c.gy);
        const int tmin = rect_min.y * c.gx + rect_min.x;
        const int tmax = ((int)rect_max.y - 1) * c.gx + (int)rect_max.x - 1;
        if (!(tmax < tmin))
            for (int rk = 0; rk < c.ws; rk++)
                if (touches_band(tmin, tmax, c.bounds[rk], c.bounds[rk + 1], c.gx, c.avoid != 0)) bits |= 1u << rk;
    }
    for (int rk = 0; rk < c.ws; rk++) {
        const uint32_t m = __ballot_sync(0xffffffffu, (bits >> rk) & 1u);
        if ((threadIdx.x & 31) == 0 && m) atomicAdd(&s_cnt[rk], __popc(m));
    }
    __syncthreads();
    if (threadIdx.x < c.ws) c.block_counts[(size_t)threadIdx.x * c.nblocks + blockIdx.x] = s_cnt[threadIdx.x];
}

__global__ void __launch_bounds__(1024)
local2j_scan_batched_kernel(const __grid_constant__ CountBatch b)
{
    const CountCamera& c = b.cam[blockIdx.y];
    if ((int)blockIdx.x >= c.ws) return;               // uniform over the CTA
    const uint32_t total = scan_row_inplace(c.block_counts + (size_t)blockIdx.x * c.nblocks, c.nblocks);
    if (threadIdx.x == 0) c.counts[blockIdx.x] = (int32_t)total;
}

struct PackOffsets {
    long long row[MAX_WS];
};

// Packs the rows selected for each destination, in ascending source index: 19 differentiable floats into `send`,
// [radius as float, depth] into `send_aux`, the source row into `send_index`.
__global__ void __launch_bounds__(PACK_TILE)
local2j_pack_kernel(int P, int gx, int gy, int ws, int nblocks, const float2* __restrict__ means2D,
                    const float* __restrict__ rgb, const float4* __restrict__ conic_opacity,
                    const float* __restrict__ means3D, const float* __restrict__ scales,
                    const float4* __restrict__ rotations, const int* __restrict__ radii,
                    const float* __restrict__ depths, const int* __restrict__ bounds, bool avoid,
                    const uint32_t* __restrict__ block_prefix, PackOffsets offs, float* __restrict__ send,
                    float* __restrict__ send_aux, int32_t* __restrict__ send_index)
{
    __shared__ uint32_t s_warp_cnt[PACK_TILE / 32];
    const int i = blockIdx.x * PACK_TILE + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t bits = 0;
    float rec[21];
    if (i < P) {
        const float2 m2 = means2D[i];
        const int rad = radii[i];
        uint2 rect_min, rect_max;
        get_rect(m2, rad, rect_min, rect_max, gx, gy);
        const int tmin = rect_min.y * gx + rect_min.x;
        const int tmax = ((int)rect_max.y - 1) * gx + (int)rect_max.x - 1;
        if (!(tmax < tmin))
            for (int rk = 0; rk < ws; rk++)
                if (touches_band(tmin, tmax, bounds[rk], bounds[rk + 1], gx, avoid)) bits |= 1u << rk;
        if (bits) {
            const float4 co = conic_opacity[i];
            const float4 q = rotations[i];
            rec[0] = m2.x; rec[1] = m2.y;
            rec[2] = rgb[3 * i]; rec[3] = rgb[3 * i + 1]; rec[4] = rgb[3 * i + 2];
            rec[5] = co.x; rec[6] = co.y; rec[7] = co.z; rec[8] = co.w;
            rec[9] = means3D[3 * i]; rec[10] = means3D[3 * i + 1]; rec[11] = means3D[3 * i + 2];
            rec[12] = scales[3 * i]; rec[13] = scales[3 * i + 1]; rec[14] = scales[3 * i + 2];
            rec[15] = q.x; rec[16] = q.y; rec[17] = q.z; rec[18] = q.w;
            rec[19] = (float)rad;
            rec[20] = depths[i];
        }
    }
    for (int rk = 0; rk < ws; rk++) {
        const bool sel = (bits >> rk) & 1u;
        const uint32_t b = __ballot_sync(0xffffffffu, sel);
        if (lane == 0) s_warp_cnt[warp] = __popc(b);
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < warp; w++) wbase += s_warp_cnt[w];
        __syncthreads();
        if (sel) {
            const long long row = offs.row[rk] + block_prefix[(size_t)rk * nblocks + blockIdx.x] + wbase +
                                  __popc(b & ((1u << lane) - 1u));
            float* dst = send + row * 19;
#pragma unroll
            for (int k = 0; k < 19; k++) dst[k] = rec[k];
            send_aux[row * 2] = rec[19];
            send_aux[row * 2 + 1] = rec[20];
            if (send_index) send_index[row] = i;
        }
    }
}

struct RowRanges {
    int n;
    long long start[MAX_WS];   // first row of range r in the gradient buffer
    long long prefix[MAX_WS + 1];  // rows in ranges before r
};

// grad rows (19 floats) of the listed row ranges are added onto the per-source-row gradient arrays.
__global__ void __launch_bounds__(256)
unpack_grad_add_kernel(RowRanges rr, const float* __restrict__ g, const int32_t* __restrict__ index,
                       float* __restrict__ d_means2D, float* __restrict__ d_rgb, float* __restrict__ d_co,
                       float* __restrict__ d_means3D, float* __restrict__ d_scales, float* __restrict__ d_rot)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total_rows = rr.prefix[rr.n];
    if (e >= total_rows * 19) return;
    const long long lrow = e / 19;
    const int c = (int)(e - lrow * 19);
    int r = 0;
    while (r + 1 < rr.n && lrow >= rr.prefix[r + 1]) r++;
    const long long row = rr.start[r] + (lrow - rr.prefix[r]);
    const size_t i = (size_t)index[row];
    const float v = g[row * 19 + c];
    if (v == 0.0f) return;
    if (c < 2) atomicAdd(d_means2D + 2 * i + c, v);
    else if (c < 5) { if (d_rgb) atomicAdd(d_rgb + 3 * i + (c - 2), v); }
    else if (c < 9) atomicAdd(d_co + 4 * i + (c - 5), v);
    else if (c < 12) { if (d_means3D) atomicAdd(d_means3D + 3 * i + (c - 9), v); }
    else if (c < 15) { if (d_scales) atomicAdd(d_scales + 3 * i + (c - 12), v); }
    else { if (d_rot) atomicAdd(d_rot + 4 * i + (c - 15), v); }
}

// Received rows arrive source-rank major; camera k's rows are one segment per source.  These two kernels move
// between that layout and the per-camera contiguous tensors the rasterizer consumes.
struct Segments {
    int n;
    long long start[MAX_WS];       // first row of segment r in the exchange buffer
    long long prefix[MAX_WS + 1];  // rows of this camera in segments before r
};

__device__ __forceinline__ long long segment_row(const Segments& sg, long long lrow)
{
    int r = 0;
    while (r + 1 < sg.n && lrow >= sg.prefix[r + 1]) r++;
    return sg.start[r] + (lrow - sg.prefix[r]);
}

__global__ void __launch_bounds__(256)
unpack_rows_kernel(Segments sg, const float* __restrict__ rows, const float* __restrict__ aux,
                   float* __restrict__ means2D, float* __restrict__ rgb, float* __restrict__ co,
                   float* __restrict__ means3D, float* __restrict__ scales, float* __restrict__ rot,
                   int* __restrict__ radii, float* __restrict__ depths)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n = sg.prefix[sg.n];
    if (e >= n * 21) return;
    const long long lrow = e / 21;
    const int c = (int)(e - lrow * 21);
    const long long row = segment_row(sg, lrow);
    if (c < 19) {
        const float v = rows[row * 19 + c];
        if (c < 2) means2D[2 * lrow + c] = v;
        else if (c < 5) rgb[3 * lrow + (c - 2)] = v;
        else if (c < 9) co[4 * lrow + (c - 5)] = v;
        else if (c < 12) means3D[3 * lrow + (c - 9)] = v;
        else if (c < 15) scales[3 * lrow + (c - 12)] = v;
        else rot[4 * lrow + (c - 15)] = v;
    } else if (c == 19) {
        radii[lrow] = (int)aux[row * 2];          // radius travels as a float, exact below 2^24
    } else {
        depths[lrow] = aux[row * 2 + 1];
    }
}

// Gradients of one camera's received tensors -> 19-float rows of the exchange buffer (NULL tensor = zeros).
__global__ void __launch_bounds__(256)
pack_grad_rows_kernel(Segments sg, const float* __restrict__ d_means2D, const float* __restrict__ d_rgb,
                      const float* __restrict__ d_co, const float* __restrict__ d_means3D,
                      const float* __restrict__ d_scales, const float* __restrict__ d_rot, float* __restrict__ rows)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n = sg.prefix[sg.n];
    if (e >= n * 19) return;
    const long long lrow = e / 19;
    const int c = (int)(e - lrow * 19);
    const long long row = segment_row(sg, lrow);
    float v = 0.f;
    if (c < 2) { if (d_means2D) v = d_means2D[2 * lrow + c]; }
    else if (c < 5) { if (d_rgb) v = d_rgb[3 * lrow + (c - 2)]; }
    else if (c < 9) { if (d_co) v = d_co[4 * lrow + (c - 5)]; }
    else if (c < 12) { if (d_means3D) v = d_means3D[3 * lrow + (c - 9)]; }
    else if (c < 15) { if (d_scales) v = d_scales[3 * lrow + (c - 12)]; }
    else { if (d_rot) v = d_rot[4 * lrow + (c - 15)]; }
    rows[row * 19 + c] = v;
}

// ---------------------------------------------------------------- peer-to-peer exchange (fused pack + transport)
// Destination tensors of one camera on one destination rank, as device pointers valid in THIS process (the
// destination's memory is mapped here; plain stores travel over NVLink).  row = first row this rank writes.
struct PeerCameraDst {
    float* means2D;
    float* rgb;
    float* conic_opacity;
    float* means3D;
    float* scales;
    float* rotations;
    int* radii;
    float* depths;
    long long row;
    float* all_map;      // plane-descriptor form of the record: replaces means3D / scales / rotations
};
struct PeerDsts {
    PeerCameraDst d[MAX_WS];
};

// Selection + packing + transport in one pass: every selected row is stored straight into the final per-camera
// tensors of the rank that renders it (its own memory for the local band), in ascending source index behind the
// rows of lower source ranks.  No send buffer, no collective, no unpack on the receiver.
// `dsts` / `local_row`: per participating rank of this camera (kernel-parameter space).  `block`: this CTA's tile.
// PLANES: the record carries the camera's plane descriptors (5 floats, read from `means3D`'s slot as a (P,5) array)
// instead of the 3-D parameters (10 floats): [m2 2 | rgb 3 | co 4 | all_map 5 | radius | depth].
template <bool PLANES>
__device__ __forceinline__ void
pack_p2p_tile(int block, int P, int gx, int gy, int ws, int nblocks, const float2* __restrict__ means2D,
              const float* __restrict__ rgb, const float4* __restrict__ conic_opacity,
              const float* __restrict__ means3D, const float* __restrict__ scales,
              const float4* __restrict__ rotations, const int* __restrict__ radii,
              const float* __restrict__ depths, const int* __restrict__ bounds, bool avoid,
              const uint32_t* __restrict__ block_prefix, const PeerCameraDst* dsts, const long long* local_row,
              int32_t* __restrict__ send_index)
{
    // The CTA's selected rows are compacted field by field in shared memory and leave as eight contiguous bursts
    // (consecutive threads store consecutive words): full-width transactions, local or across NVLink.
    __shared__ uint32_t s_warp_cnt[PACK_TILE / 32];
    constexpr int NF = PLANES ? 16 : 21;       // staged fields; the last two are radius and depth
    __shared__ float s_f[NF][PACK_TILE + 1];   // field-major staging: [m2 2 | rgb 3 | co 4 | m3 3 | sc 3 | rot 4 | radius | depth]
    const int i = block * PACK_TILE + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t bits = 0;
    float rec[NF];
    if (i < P) {
        const float2 m2 = means2D[i];
        const int rad = radii[i];
        uint2 rect_min, rect_max;
        get_rect(m2, rad, rect_min, rect_max, gx, gy);
        const int tmin = rect_min.y * gx + rect_min.x;
        const int tmax = ((int)rect_max.y - 1) * gx + (int)rect_max.x - 1;
        if (!(tmax < tmin))
            for (int rk = 0; rk < ws; rk++)
                if (touches_band(tmin, tmax, bounds[rk], bounds[rk + 1], gx, avoid)) bits |= 1u << rk;
        if (bits) {
            const float4 co = conic_opacity[i];
            rec[0] = m2.x; rec[1] = m2.y;
            rec[2] = rgb[3 * i]; rec[3] = rgb[3 * i + 1]; rec[4] = rgb[3 * i + 2];
            rec[5] = co.x; rec[6] = co.y; rec[7] = co.z; rec[8] = co.w;
            if (PLANES) {
#pragma unroll
                for (int k = 0; k < 5; k++) rec[9 + k] = means3D[5 * (size_t)i + k];
            } else {
                const float4 q = rotations[i];
                rec[9] = means3D[3 * i]; rec[10] = means3D[3 * i + 1]; rec[11] = means3D[3 * i + 2];
                rec[12] = scales[3 * i]; rec[13] = scales[3 * i + 1]; rec[14] = scales[3 * i + 2];
                rec[15] = q.x; rec[16] = q.y; rec[17] = q.z; rec[18] = q.w;
            }
            rec[NF - 2] = __int_as_float(rad);
            rec[NF - 1] = depths[i];
        }
    }
    if (!__syncthreads_or(bits != 0)) return;   // nothing of this tile is visible to any rank (uniform over the CTA)
    for (int rk = 0; rk < ws; rk++) {
        const bool sel = (bits >> rk) & 1u;
        const uint32_t b = __ballot_sync(0xffffffffu, sel);
        if (lane == 0) s_warp_cnt[warp] = __popc(b);
        __syncthreads();
        uint32_t wbase = 0, cnt = 0;
        for (int w = 0; w < PACK_TILE / 32; w++) {
            if (w < warp) wbase += s_warp_cnt[w];
            cnt += s_warp_cnt[w];
        }
        if (cnt == 0) {          // uniform over the CTA
            __syncthreads();
            continue;
        }
        const uint32_t slot = wbase + __popc(b & ((1u << lane) - 1u));
        const long long seg0 = (long long)block_prefix[(size_t)rk * nblocks + block];
        if (sel) {
#pragma unroll
            for (int k = 0; k < NF; k++) s_f[k][slot] = rec[k];
            if (send_index) send_index[local_row[rk] + seg0 + slot] = i;
        }
        __syncthreads();
        const PeerCameraDst& D = dsts[rk];
        const long long row0 = D.row + seg0;
        // field f of width w occupies words [row0*w, (row0+cnt)*w) of its destination array
        auto burst = [&](float* dst, int f0, int w) {
            const int n = (int)cnt * w;
            float* out = dst + row0 * w;
            for (int e = threadIdx.x; e < n; e += PACK_TILE) out[e] = s_f[f0 + e % w][e / w];
        };
        burst(D.means2D, 0, 2);
        burst(D.rgb, 2, 3);
        burst(D.conic_opacity, 5, 4);
        if (PLANES) {
            burst(D.all_map, 9, 5);
        } else {
            burst(D.means3D, 9, 3);
            burst(D.scales, 12, 3);
            burst(D.rotations, 15, 4);
        }
        for (int e = threadIdx.x; e < (int)cnt; e += PACK_TILE) {
            D.radii[row0 + e] = __float_as_int(s_f[NF - 2][e]);
            D.depths[row0 + e] = s_f[NF - 1][e];
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(PACK_TILE)
local2j_pack_p2p_kernel(int P, int gx, int gy, int ws, int nblocks, const float2* __restrict__ means2D,
                        const float* __restrict__ rgb, const float4* __restrict__ conic_opacity,
                        const float* __restrict__ means3D, const float* __restrict__ scales,
                        const float4* __restrict__ rotations, const int* __restrict__ radii,
                        const float* __restrict__ depths, const int* __restrict__ bounds, bool avoid,
                        const uint32_t* __restrict__ block_prefix, const __grid_constant__ PeerDsts dsts,
                        const __grid_constant__ PackOffsets local_offs, int32_t* __restrict__ send_index)
{
    pack_p2p_tile<false>(blockIdx.x, P, gx, gy, ws, nblocks, means2D, rgb, conic_opacity, means3D, scales, rotations,
                         radii, depths, bounds, avoid, block_prefix, dsts.d, local_offs.row, send_index);
}

// All cameras of a batch in one launch: blockIdx.y = camera, blockIdx.x = tile of that camera's local Gaussians.
constexpr int MAX_XCAMS = 16;      // cameras per launch
constexpr int MAX_XENTRIES = 48;   // participating (camera, rank) pairs per launch: cuts are contiguous, so a batch
                                   // of B cameras over ws ranks has at most B + ws - 1 of them
struct ExchangeCamera {
    const float2* means2D;
    const float* rgb;
    const float4* conic_opacity;
    const float* means3D;
    const float* scales;
    const float4* rotations;
    const int* radii;
    const float* depths;
    const int* bounds;
    const uint32_t* block_prefix;
    int P, gx, gy, ws, nblocks, avoid, entry0, pad;
};
struct ExchangeBatch {
    ExchangeCamera cam[MAX_XCAMS];
    PeerCameraDst dst[MAX_XENTRIES];
    long long local_row[MAX_XENTRIES];
};

template <bool PLANES>
__global__ void __launch_bounds__(PACK_TILE)
local2j_pack_p2p_batched_kernel(const __grid_constant__ ExchangeBatch b, int32_t* __restrict__ send_index)
{
    const ExchangeCamera& c = b.cam[blockIdx.y];
    if ((int)blockIdx.x >= c.nblocks) return;          // uniform over the CTA
    pack_p2p_tile<PLANES>(blockIdx.x, c.P, c.gx, c.gy, c.ws, c.nblocks, c.means2D, c.rgb, c.conic_opacity, c.means3D,
                          c.scales, c.rotations, c.radii, c.depths, c.bounds, c.avoid != 0, c.block_prefix,
                          b.dst + c.entry0, b.local_row + c.entry0, send_index);
}

struct GradSegments {
    int n;
    float* rows[MAX_WS];           // where segment r's 19-float gradient rows go (possibly another GPU's memory)
    long long prefix[MAX_WS + 1];  // rows of this camera in segments before r
    long long first_row;           // the grid starts at this row and wraps around: ranks that start at different
                                   // segments do not all store into the same peer at the same time
};

// NCOLS = 19: all differentiable columns; NCOLS = 9: only means2D | rgb | conic_opacity (the 3-D parameters carry
// no gradient back when the receiver builds its plane descriptors without autograd); NCOLS = 14: means2D | rgb |
// conic_opacity | plane descriptors (5), whose (n,5) array is passed in the means3D argument.
template <int NCOLS>
__global__ void __launch_bounds__(256)
pack_grad_rows_to_kernel(GradSegments sg, const float* __restrict__ d_means2D, const float* __restrict__ d_rgb,
                         const float* __restrict__ d_co, const float* __restrict__ d_means3D,
                         const float* __restrict__ d_scales, const float* __restrict__ d_rot)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n = sg.prefix[sg.n];
    if (e >= n * NCOLS) return;
    const long long lrow0 = e / NCOLS;
    const int c = (int)(e - lrow0 * NCOLS);
    long long lrow = lrow0 + sg.first_row;
    if (lrow >= n) lrow -= n;
    int r = 0;
    while (r + 1 < sg.n && lrow >= sg.prefix[r + 1]) r++;
    float v = 0.f;
    if (c < 2) { if (d_means2D) v = d_means2D[2 * lrow + c]; }
    else if (c < 5) { if (d_rgb) v = d_rgb[3 * lrow + (c - 2)]; }
    else if (c < 9) { if (d_co) v = d_co[4 * lrow + (c - 5)]; }
    else if (NCOLS == 14) { if (d_means3D) v = d_means3D[5 * lrow + (c - 9)]; }     // plane descriptors (n,5)
    else if (c < 12) { if (d_means3D) v = d_means3D[3 * lrow + (c - 9)]; }
    else if (c < 15) { if (d_scales) v = d_scales[3 * lrow + (c - 12)]; }
    else { if (d_rot) v = d_rot[4 * lrow + (c - 15)]; }
    sg.rows[r][(lrow - sg.prefix[r]) * NCOLS + c] = v;
}

template <int NCOLS>
__global__ void __launch_bounds__(256)
unpack_grad_add_cols_kernel(RowRanges rr, const float* __restrict__ g, const int32_t* __restrict__ index,
                            float* __restrict__ d_means2D, float* __restrict__ d_rgb, float* __restrict__ d_co,
                            float* __restrict__ d_means3D, float* __restrict__ d_scales, float* __restrict__ d_rot)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total_rows = rr.prefix[rr.n];
    if (e >= total_rows * NCOLS) return;
    const long long lrow = e / NCOLS;
    const int c = (int)(e - lrow * NCOLS);
    int r = 0;
    while (r + 1 < rr.n && lrow >= rr.prefix[r + 1]) r++;
    const long long row = rr.start[r] + (lrow - rr.prefix[r]);
    const size_t i = (size_t)index[row];
    const float v = g[row * NCOLS + c];
    if (v == 0.0f) return;
    if (c < 2) atomicAdd(d_means2D + 2 * i + c, v);
    else if (c < 5) { if (d_rgb) atomicAdd(d_rgb + 3 * i + (c - 2), v); }
    else if (c < 9) atomicAdd(d_co + 4 * i + (c - 5), v);
    else if (NCOLS == 14) { if (d_means3D) atomicAdd(d_means3D + 5 * i + (c - 9), v); }   // plane descriptors (P,5)
    else if (c < 12) { if (d_means3D) atomicAdd(d_means3D + 3 * i + (c - 9), v); }
    else if (c < 15) { if (d_scales) atomicAdd(d_scales + 3 * i + (c - 12), v); }
    else { if (d_rot) atomicAdd(d_rot + 4 * i + (c - 15), v); }
}

}  // namespace cgx

using namespace cgx;

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

extern "C" uint32_t cgx_higher_msb(uint32_t n)
{
    uint32_t msb = sizeof(n) * 4;
    uint32_t step = msb;
    while (step > 1) {
        step /= 2;
        if (n >> msb)
            msb += step;
        else
            msb -= step;
    }
    if (n >> msb) msb++;
    return msb;
}

// CTA partial sums, then the analysed mask (MaskBand) on the next 256-byte boundary
static size_t bin_band_offset(int P)
{
    const size_t nblocks = ((size_t)(P > 0 ? P : 1) + SCAN_TILE - 1) / SCAN_TILE;
    return align_up(nblocks * sizeof(uint32_t), 256);
}

// ... then the per-CTA depth ranges (two words per CTA)
extern "C" size_t cgx_bin_workspace_bytes(int P)
{
    const size_t nblocks = ((size_t)(P > 0 ? P : 1) + SCAN_TILE - 1) / SCAN_TILE;
    return bin_band_offset(P) + 256 + align_up(2 * nblocks * sizeof(uint32_t), 256);
}

static int bin_count_scan(int P, int W, int H, const int32_t* radii, const float* means2D, const float* depths,
                          const uint8_t* compute_locally, uint32_t* tiles_touched, uint32_t* num_rendered,
                          void* workspace, size_t workspace_bytes, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0 || !num_rendered) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if (P == 0) {
        cudaError_t e = cudaMemsetAsync(num_rendered, 0, (depths ? 3 : 1) * sizeof(uint32_t), st);
        if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
        return CGX_OK;
    }
    if (!radii || !means2D || !compute_locally || !tiles_touched || !workspace) return CGX_EINVAL;
    if ((uintptr_t)means2D & 7) return CGX_EINVAL;
    if (workspace_bytes < cgx_bin_workspace_bytes(P)) return CGX_ENOMEM;
    const int gx = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, gy = (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
    const int nblocks = (P + SCAN_TILE - 1) / SCAN_TILE;
    uint32_t* sums = (uint32_t*)workspace;
    MaskBand* band = (MaskBand*)((char*)workspace + bin_band_offset(P));
    uint32_t* block_ranges = depths ? (uint32_t*)((char*)workspace + bin_band_offset(P) + 256) : nullptr;
    analyse_mask_kernel<<<1, 1024, 0, st>>>(gx, gy, compute_locally, band);
    const int vec_ok = aligned16(radii) && aligned16(means2D) && aligned16(tiles_touched) && (!depths || aligned16(depths));
    tile_count_kernel<<<nblocks, CGX_BLOCK_SIZE, 0, st>>>(P, gx, gy, radii, (const float2*)means2D, compute_locally,
                                                          tiles_touched, sums, band, depths, block_ranges, vec_ok);
    scan_partials_kernel<<<1, 1024, 0, st>>>(nblocks, sums, num_rendered, block_ranges);
    return check_launch(3);
}

extern "C" int cgx_bin_count_scan(int P, int W, int H, const int32_t* radii, const float* means2D,
                                  const uint8_t* compute_locally, uint32_t* tiles_touched, uint32_t* num_rendered,
                                  void* workspace, size_t workspace_bytes, void* stream)
{
    return bin_count_scan(P, W, H, radii, means2D, nullptr, compute_locally, tiles_touched, num_rendered, workspace,
                          workspace_bytes, stream);
}

extern "C" int cgx_bin_count_scan_depths(int P, int W, int H, const int32_t* radii, const float* means2D,
                                         const float* depths, const uint8_t* compute_locally, uint32_t* tiles_touched,
                                         uint32_t* num_rendered3, void* workspace, size_t workspace_bytes, void* stream)
{
    if (P > 0 && !depths) return CGX_EINVAL;
    return bin_count_scan(P, W, H, radii, means2D, depths, compute_locally, tiles_touched, num_rendered3, workspace,
                          workspace_bytes, stream);
}

extern "C" int cgx_emit_keys(int P, int W, int H, const int32_t* radii, const float* means2D, const float* depths,
                             const uint32_t* tiles_touched, const uint8_t* compute_locally, uint32_t* point_offsets,
                             uint64_t* keys, uint32_t* values, int64_t capacity, const void* workspace, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0 || capacity < 0 || capacity > 0xffffffffLL) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!radii || !means2D || !depths || !tiles_touched || !compute_locally || !point_offsets || !workspace)
        return CGX_EINVAL;
    if (capacity > 0 && (!keys || !values)) return CGX_EINVAL;
    const int gx = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, gy = (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
    const int nblocks = (P + SCAN_TILE - 1) / SCAN_TILE;
    emit_keys_kernel<<<nblocks, CGX_BLOCK_SIZE, 0, (cudaStream_t)stream>>>(
        P, gx, gy, radii, (const float2*)means2D, depths, tiles_touched, compute_locally, (const uint32_t*)workspace,
        point_offsets, keys, values, (uint32_t)capacity,
        (const MaskBand*)((const char*)workspace + bin_band_offset(P)),
        aligned16(tiles_touched) && aligned16(point_offsets) ? 1 : 0);
    return check_launch();
}

static int g_sort_variant = -1;  // test-only switch: -1 three-kernel passes, scatter chosen by size (default);
                                 // 0 staged scatter; 1 unstaged scatter; 2 one-sweep passes

extern "C" int cgx_set_sort_variant(int variant)
{
    g_sort_variant = variant;
    return CGX_OK;
}

extern "C" int cgx_sort_passes(int end_bit) { return end_bit <= 0 ? 0 : (end_bit + RADIX_BITS - 1) / RADIX_BITS; }

static size_t legacy_sort_bytes(int64_t n)
{
    const size_t nblocks = ((size_t)(n > 0 ? n : 1) + SORT_TILE - 1) / SORT_TILE;
    return align_up(nblocks * RADIX * sizeof(uint32_t), 256) + align_up(RADIX * sizeof(uint32_t), 256);
}

static size_t onesweep_head_bytes() { return align_up(OS_MAX_PASSES * RADIX * sizeof(uint32_t), 256) + 256; }

static size_t onesweep_sort_bytes(int64_t n, int passes)
{
    const size_t ntiles = ((size_t)(n > 0 ? n : 1) + OS_TILE - 1) / OS_TILE;
    return onesweep_head_bytes() + (size_t)passes * ntiles * RADIX * sizeof(uint32_t);
}

extern "C" size_t cgx_sort_workspace_bytes(int64_t n)
{
    const size_t a = legacy_sort_bytes(n), b = onesweep_sort_bytes(n, OS_MAX_PASSES);
    return a > b ? a : b;
}

namespace cgx {
int fetch_sort_status_async(int* out_pinned, cudaStream_t st)
{
    void* word = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&word, g_sort_status);
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    return post_words(word, out_pinned, 1, st);
}
int fetch_sort_status(int* out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, g_sort_status, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    if (*out != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_sort_status, &zero, sizeof(int));
    }
    return CGX_OK;
}
}  // namespace cgx

// The pairs start in (ka, va).  After `passes` passes they are in (ka, va) when `passes` is even, else in (kb, vb).
// variant: see g_sort_variant; the one-sweep path needs onesweep_sort_bytes(n, passes) of workspace.
static int sort_passes_run(int variant, int64_t n, int end_bit, int low_bits, uint64_t* ka, uint32_t* va, uint64_t* kb,
                           uint32_t* vb, void* workspace, size_t workspace_bytes, unsigned long long wait_limit,
                           cudaStream_t st)
{
    // bits [low_bits, 32) are equal in all keys: the sort runs over the squeezed key of end_bit - (32 - low_bits) bits
    if (low_bits < 0 || low_bits > 32) return CGX_EINVAL;
    if (end_bit <= 32) low_bits = 32;
    end_bit -= 32 - low_bits;
    const int passes = cgx_sort_passes(end_bit);
    if (passes == 0) return CGX_OK;
    uint64_t *kin = ka, *kout = kb;
    uint32_t *vin = va, *vout = vb;
    const bool onesweep = variant == 2 && passes <= OS_MAX_PASSES && n < ((int64_t)1 << 30) &&
                          workspace_bytes >= onesweep_sort_bytes(n, passes);
    if (onesweep) {
        const int ntiles = (int)((n + OS_TILE - 1) / OS_TILE);
        uint32_t* ghist = (uint32_t*)workspace;
        uint32_t* tickets = (uint32_t*)((char*)workspace + align_up(OS_MAX_PASSES * RADIX * sizeof(uint32_t), 256));
        uint32_t* status = (uint32_t*)((char*)workspace + onesweep_head_bytes());
        cudaError_t e = cudaMemsetAsync(workspace, 0, onesweep_sort_bytes(n, passes), st);
        if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
        const int hist_grid = ntiles < 148 * 8 ? ntiles : 148 * 8;
        os_hist_kernel<<<hist_grid, OS_THREADS, 0, st>>>(n, passes, end_bit, low_bits, kin, ghist);
        for (int p = 0; p < passes; p++) {
            const int shift = p * RADIX_BITS;
            const int bits = (end_bit - shift) < RADIX_BITS ? (end_bit - shift) : RADIX_BITS;
            os_pass_kernel<<<ntiles, OS_THREADS, 0, st>>>(n, digit_spec(shift, (1u << bits) - 1u, low_bits), kin, vin, kout, vout,
                                                         ghist + p * RADIX, tickets + p,
                                                         status + (size_t)p * ntiles * RADIX,
                                                         wait_limit ? wait_limit : OS_WAIT_LIMIT_CYCLES);
            uint64_t* tk = kin; kin = kout; kout = tk;
            uint32_t* tv = vin; vin = vout; vout = tv;
        }
        return check_launch(1 + passes);
    }
    if (workspace_bytes < legacy_sort_bytes(n)) return CGX_ENOMEM;
    {
        // opt in to > 48 KB of dynamic shared memory (per device, cheap and idempotent)
        cudaError_t e = cudaFuncSetAttribute(sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SORT_SMEM);
        if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    }
    const int nblocks = (int)((n + SORT_TILE - 1) / SORT_TILE);
    // both ping-pong buffers in L2 -> unstaged scatter; otherwise stage each tile so digit runs leave as bursts
    const bool direct = variant == 1 || (variant != 0 && n * 24 <= (int64_t)96 << 20);
    uint32_t* table = (uint32_t*)workspace;
    uint32_t* totals = (uint32_t*)((char*)workspace + align_up((size_t)nblocks * RADIX * sizeof(uint32_t), 256));
    for (int p = 0; p < passes; p++) {
        const int shift = p * RADIX_BITS;
        const int bits = (end_bit - shift) < RADIX_BITS ? (end_bit - shift) : RADIX_BITS;
        const uint32_t mask = (1u << bits) - 1u;
        const DigitSpec dg = digit_spec(shift, mask, low_bits);
        sort_hist_kernel<<<nblocks, SORT_THREADS, 0, st>>>(n, nblocks, dg, kin, table);
        sort_scan_rows_kernel<<<RADIX, 1024, 0, st>>>(nblocks, table, totals);
        if (direct)
            sort_scatter_direct_kernel<<<nblocks, SORT_THREADS, 0, st>>>(n, nblocks, dg, kin, vin, kout, vout,
                                                                        table, totals);
        else
            sort_scatter_kernel<<<nblocks, SORT_THREADS, SORT_SMEM, st>>>(n, nblocks, dg, kin, vin, kout, vout,
                                                                         table, totals);
        uint64_t* tk = kin; kin = kout; kout = tk;
        uint32_t* tv = vin; vin = vout; vout = tv;
    }
    return check_launch(3 * passes);
}

static int sort_pairs_into_out(int variant, int64_t n, int end_bit, uint64_t* keys_in, uint32_t* values_in,
                               uint64_t* keys_out, uint32_t* values_out, void* workspace, size_t workspace_bytes,
                               void* stream)
{
    if (n < 0 || end_bit < 0 || end_bit > 64 || n > 0x7fffffffLL) return CGX_EINVAL;
    if (n == 0) return CGX_OK;
    if (!keys_in || !values_in || !keys_out || !values_out || !workspace) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    const int passes = cgx_sort_passes(end_bit);
    if (passes % 2 == 0) {
        // an even number of passes ends where it started: start from `out` (callers that own both buffers avoid
        // this copy with cgx_sort_pairs_pingpong)
        cudaMemcpyAsync(keys_out, keys_in, n * sizeof(uint64_t), cudaMemcpyDeviceToDevice, st);
        cudaMemcpyAsync(values_out, values_in, n * sizeof(uint32_t), cudaMemcpyDeviceToDevice, st);
        if (passes == 0) return check_launch(0);
        return sort_passes_run(variant, n, end_bit, 32, keys_out, values_out, keys_in, values_in, workspace,
                               workspace_bytes, 0ull, st);
    }
    return sort_passes_run(variant, n, end_bit, 32, keys_in, values_in, keys_out, values_out, workspace,
                           workspace_bytes, 0ull, st);
}

extern "C" int cgx_sort_pairs(int64_t n, int end_bit, uint64_t* keys_in, uint32_t* values_in, uint64_t* keys_out,
                              uint32_t* values_out, void* workspace, size_t workspace_bytes, void* stream)
{
    if (n > 0 && workspace && workspace_bytes < legacy_sort_bytes(n) &&
        workspace_bytes < onesweep_sort_bytes(n, cgx_sort_passes(end_bit)))
        return CGX_ENOMEM;
    return sort_pairs_into_out(g_sort_variant, n, end_bit, keys_in, values_in, keys_out, values_out, workspace,
                               workspace_bytes, stream);
}

extern "C" int cgx_sort_pairs_pingpong(int64_t n, int end_bit, int low_bits, uint64_t* keys_a, uint32_t* values_a,
                                       uint64_t* keys_b, uint32_t* values_b, void* workspace, size_t workspace_bytes,
                                       unsigned long long wait_limit_cycles, void* stream)
{
    if (n < 0 || end_bit < 0 || end_bit > 64 || n > 0x7fffffffLL || low_bits < 0 || low_bits > 32) return CGX_EINVAL;
    if (n == 0) return CGX_OK;
    if (!keys_a || !values_a || !keys_b || !values_b || !workspace) return CGX_EINVAL;
    if (workspace_bytes < legacy_sort_bytes(n) && workspace_bytes < onesweep_sort_bytes(n, cgx_sort_passes(end_bit)))
        return CGX_ENOMEM;
    return sort_passes_run(g_sort_variant, n, end_bit, low_bits, keys_a, values_a, keys_b, values_b, workspace,
                           workspace_bytes, wait_limit_cycles, (cudaStream_t)stream);
}

extern "C" int cgx_tile_ranges(int64_t n, int T, const uint64_t* keys_sorted, uint32_t* ranges, void* stream)
{
    if (n < 0 || T <= 0 || !ranges) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(ranges, 0, (size_t)T * sizeof(uint2), st);
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    if (n == 0) return CGX_OK;
    if (!keys_sorted) return CGX_EINVAL;
    tile_ranges_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(n, (uint32_t)T, keys_sorted, (uint2*)ranges);
    return check_launch();
}

extern "C" int cgx_local2j_mask(int P, int H, int W, int ws, const float* means2D, const int32_t* radii,
                                const int32_t* tile_bounds, int avoid_pixel_all2all, uint8_t* mask, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0 || ws <= 0) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means2D || !radii || !tile_bounds || !mask || ((uintptr_t)means2D & 7)) return CGX_EINVAL;
    const int gx = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, gy = (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
    local2j_mask_kernel<<<(P + 255) / 256, 256, 0, (cudaStream_t)stream>>>(P, gx, gy, ws, (const float2*)means2D, radii,
                                                                          tile_bounds, avoid_pixel_all2all != 0, mask);
    return check_launch();
}

extern "C" size_t cgx_local2j_workspace_bytes(int P, int ws)
{
    const size_t nblocks = ((size_t)(P > 0 ? P : 1) + PACK_TILE - 1) / PACK_TILE;
    return align_up(nblocks * (size_t)(ws > 0 ? ws : 1) * sizeof(uint32_t), 256);
}

extern "C" int cgx_local2j_count(int P, int H, int W, int ws, const float* means2D, const int32_t* radii,
                                 const int32_t* tile_bounds, int avoid_pixel_all2all, int32_t* counts,
                                 void* workspace, size_t workspace_bytes, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0 || ws <= 0 || ws > MAX_WS || !counts) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if (P == 0) {
        cudaError_t e = cudaMemsetAsync(counts, 0, ws * sizeof(int32_t), st);
        if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
        return CGX_OK;
    }
    if (!means2D || !radii || !tile_bounds || !workspace || ((uintptr_t)means2D & 7)) return CGX_EINVAL;
    if (workspace_bytes < cgx_local2j_workspace_bytes(P, ws)) return CGX_ENOMEM;
    const int gx = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, gy = (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
    const int nblocks = (P + PACK_TILE - 1) / PACK_TILE;
    local2j_count_kernel<<<nblocks, PACK_TILE, 0, st>>>(P, gx, gy, ws, nblocks, (const float2*)means2D, radii,
                                                        tile_bounds, avoid_pixel_all2all != 0, (uint32_t*)workspace);
    local2j_scan_kernel<<<ws, 1024, 0, st>>>(nblocks, (uint32_t*)workspace, counts);
    return check_launch(2);
}

extern "C" int cgx_local2j_count_batched(int n_cameras, const cgx_count_camera* cams, void* stream)
{
    if (n_cameras < 0 || (n_cameras > 0 && !cams)) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    int k0 = 0;
    while (k0 < n_cameras) {
        CountBatch b;
        memset(&b, 0, sizeof(b));
        int n = 0, max_blocks = 0, max_ws = 0;
        for (; k0 + n < n_cameras && n < MAX_COUNT_CAMS; n++) {
            const cgx_count_camera& c = cams[k0 + n];
            if (c.P < 0 || c.W <= 0 || c.H <= 0 || c.ws <= 0 || c.ws > MAX_WS || !c.counts) return CGX_EINVAL;
            CountCamera& x = b.cam[n];
            x.P = (int)c.P;
            x.ws = (int)c.ws;
            x.gx = ((int)c.W + CGX_BLOCK_X - 1) / CGX_BLOCK_X;
            x.gy = ((int)c.H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
            x.nblocks = (x.P + PACK_TILE - 1) / PACK_TILE;
            x.avoid = c.avoid_pixel_all2all != 0;
            x.counts = c.counts;
            if (x.P == 0) {
                cudaError_t e = cudaMemsetAsync(c.counts, 0, x.ws * sizeof(int32_t), st);
                if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
                x.ws = 0;                      // nothing to scan for this camera
                continue;
            }
            if (!c.means2D || !c.radii || !c.tile_bounds || !c.workspace || ((uintptr_t)c.means2D & 7)) return CGX_EINVAL;
            if ((size_t)c.workspace_bytes < cgx_local2j_workspace_bytes(x.P, x.ws)) return CGX_ENOMEM;
            x.means2D = (const float2*)c.means2D;
            x.radii = c.radii;
            x.bounds = c.tile_bounds;
            x.block_counts = (uint32_t*)c.workspace;
            if (x.nblocks > max_blocks) max_blocks = x.nblocks;
            if (x.ws > max_ws) max_ws = x.ws;
        }
        if (max_blocks > 0) {
            local2j_count_batched_kernel<<<dim3((unsigned)max_blocks, (unsigned)n), PACK_TILE, 0, st>>>(b);
            local2j_scan_batched_kernel<<<dim3((unsigned)max_ws, (unsigned)n), 1024, 0, st>>>(b);
            const int rc = check_launch(2);
            if (rc != CGX_OK) return rc;
        }
        k0 += n;
    }
    return CGX_OK;
}

extern "C" int cgx_local2j_pack(int P, int H, int W, int ws, const float* means2D, const float* rgb,
                                const float* conic_opacity, const float* means3D, const float* scales,
                                const float* rotations, const int32_t* radii, const float* depths,
                                const int32_t* tile_bounds, int avoid_pixel_all2all, const int64_t* send_row_offset,
                                float* send_buffer, float* send_aux, int32_t* send_index, void* workspace,
                                size_t workspace_bytes, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0 || ws <= 0 || ws > MAX_WS || !send_row_offset) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means2D || !rgb || !conic_opacity || !means3D || !scales || !rotations || !radii || !depths ||
        !tile_bounds || !send_buffer || !send_aux || !workspace)
        return CGX_EINVAL;
    if (((uintptr_t)means2D & 7) || !aligned16(conic_opacity) || !aligned16(rotations)) return CGX_EINVAL;
    if (workspace_bytes < cgx_local2j_workspace_bytes(P, ws)) return CGX_ENOMEM;
    const int gx = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, gy = (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
    const int nblocks = (P + PACK_TILE - 1) / PACK_TILE;
    PackOffsets offs;
    for (int j = 0; j < MAX_WS; j++) offs.row[j] = j < ws ? (long long)send_row_offset[j] : 0;
    local2j_pack_kernel<<<nblocks, PACK_TILE, 0, (cudaStream_t)stream>>>(
        P, gx, gy, ws, nblocks, (const float2*)means2D, rgb, (const float4*)conic_opacity, means3D, scales,
        (const float4*)rotations, radii, depths, tile_bounds, avoid_pixel_all2all != 0, (const uint32_t*)workspace, offs,
        send_buffer, send_aux, send_index);
    return check_launch();
}

extern "C" int cgx_unpack_grad_add(int n_ranges, const int64_t* range_start, const int64_t* range_stop,
                                   const float* grad_rows, const int32_t* send_index, float* d_means2D, float* d_rgb,
                                   float* d_conic_opacity, float* d_means3D, float* d_scales, float* d_rotations,
                                   void* stream)
{
    if (n_ranges < 0 || n_ranges > MAX_WS) return CGX_EINVAL;
    if (n_ranges == 0) return CGX_OK;
    if (!range_start || !range_stop) return CGX_EINVAL;
    RowRanges rr;
    rr.n = n_ranges;
    rr.prefix[0] = 0;
    for (int r = 0; r < n_ranges; r++) {
        if (range_stop[r] < range_start[r] || range_start[r] < 0) return CGX_EINVAL;
        rr.start[r] = range_start[r];
        rr.prefix[r + 1] = rr.prefix[r] + (range_stop[r] - range_start[r]);
    }
    const long long total = rr.prefix[n_ranges] * 19;
    if (total == 0) return CGX_OK;
    if (!grad_rows || !send_index || !d_means2D || !d_conic_opacity) return CGX_EINVAL;
    unpack_grad_add_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        rr, grad_rows, send_index, d_means2D, d_rgb, d_conic_opacity, d_means3D, d_scales, d_rotations);
    return check_launch();
}

static int fill_segments(Segments& sg, int n_segments, const int64_t* seg_start, const int64_t* seg_count)
{
    if (n_segments < 0 || n_segments > MAX_WS) return CGX_EINVAL;
    if (n_segments > 0 && (!seg_start || !seg_count)) return CGX_EINVAL;
    sg.n = n_segments;
    sg.prefix[0] = 0;
    for (int r = 0; r < n_segments; r++) {
        if (seg_start[r] < 0 || seg_count[r] < 0) return CGX_EINVAL;
        sg.start[r] = seg_start[r];
        sg.prefix[r + 1] = sg.prefix[r] + seg_count[r];
    }
    return CGX_OK;
}

extern "C" int cgx_unpack_rows(int n_segments, const int64_t* seg_start, const int64_t* seg_count, const float* rows,
                               const float* aux, float* means2D, float* rgb, float* conic_opacity, float* means3D,
                               float* scales, float* rotations, int32_t* radii, float* depths, void* stream)
{
    Segments sg;
    int st = fill_segments(sg, n_segments, seg_start, seg_count);
    if (st != CGX_OK) return st;
    const long long n = n_segments ? sg.prefix[n_segments] : 0;
    if (n == 0) return CGX_OK;
    if (!rows || !aux || !means2D || !rgb || !conic_opacity || !means3D || !scales || !rotations || !radii || !depths)
        return CGX_EINVAL;
    unpack_rows_kernel<<<(unsigned)((n * 21 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        sg, rows, aux, means2D, rgb, conic_opacity, means3D, scales, rotations, radii, depths);
    return check_launch();
}

extern "C" int cgx_pack_grad_rows(int n_segments, const int64_t* seg_start, const int64_t* seg_count,
                                  const float* d_means2D, const float* d_rgb, const float* d_conic_opacity,
                                  const float* d_means3D, const float* d_scales, const float* d_rotations, float* rows,
                                  void* stream)
{
    Segments sg;
    int st = fill_segments(sg, n_segments, seg_start, seg_count);
    if (st != CGX_OK) return st;
    const long long n = n_segments ? sg.prefix[n_segments] : 0;
    if (n == 0) return CGX_OK;
    if (!rows) return CGX_EINVAL;
    pack_grad_rows_kernel<<<(unsigned)((n * 19 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        sg, d_means2D, d_rgb, d_conic_opacity, d_means3D, d_scales, d_rotations, rows);
    return check_launch();
}

extern "C" int cgx_local2j_pack_p2p(int P, int H, int W, int ws, const float* means2D, const float* rgb,
                                    const float* conic_opacity, const float* means3D, const float* scales,
                                    const float* rotations, const int32_t* radii, const float* depths,
                                    const int32_t* tile_bounds, int avoid_pixel_all2all,
                                    const cgx_peer_camera_dst* dst, const int64_t* send_row_offset,
                                    int32_t* send_index, void* workspace, size_t workspace_bytes, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0 || ws <= 0 || ws > MAX_WS || !dst) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means2D || !rgb || !conic_opacity || !means3D || !scales || !rotations || !radii || !depths ||
        !tile_bounds || !workspace)
        return CGX_EINVAL;
    if (send_index && !send_row_offset) return CGX_EINVAL;
    if (((uintptr_t)means2D & 7) || !aligned16(conic_opacity) || !aligned16(rotations)) return CGX_EINVAL;
    if (workspace_bytes < cgx_local2j_workspace_bytes(P, ws)) return CGX_ENOMEM;
    PeerDsts dsts;
    PackOffsets offs;
    for (int j = 0; j < MAX_WS; j++) {
        offs.row[j] = (j < ws && send_row_offset) ? (long long)send_row_offset[j] : 0;
        if (j >= ws) {
            dsts.d[j] = PeerCameraDst{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, nullptr};
            continue;
        }
        const cgx_peer_camera_dst& s = dst[j];
        if (!s.means2D || !s.rgb || !s.conic_opacity || !s.means3D || !s.scales || !s.rotations || !s.radii ||
            !s.depths || s.first_row < 0)
            return CGX_EINVAL;
        if (((uintptr_t)s.means2D & 7) || !aligned16(s.conic_opacity) || !aligned16(s.rotations)) return CGX_EINVAL;
        dsts.d[j] = PeerCameraDst{s.means2D, s.rgb, s.conic_opacity, s.means3D, s.scales, s.rotations, s.radii,
                                  s.depths, (long long)s.first_row, nullptr};
    }
    const int gx = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, gy = (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
    const int nblocks = (P + PACK_TILE - 1) / PACK_TILE;
    local2j_pack_p2p_kernel<<<nblocks, PACK_TILE, 0, (cudaStream_t)stream>>>(
        P, gx, gy, ws, nblocks, (const float2*)means2D, rgb, (const float4*)conic_opacity, means3D, scales,
        (const float4*)rotations, radii, depths, tile_bounds, avoid_pixel_all2all != 0, (const uint32_t*)workspace, dsts,
        offs, send_index);
    return check_launch();
}

extern "C" int cgx_local2j_pack_p2p_batched(int n_cameras, const cgx_exchange_camera* cams, int32_t* send_index,
                                            void* stream)
{
    if (n_cameras < 0 || (n_cameras > 0 && !cams)) return CGX_EINVAL;
    const bool planes = n_cameras > 0 && cams[0].all_map != nullptr;
    for (int k = 0; k < n_cameras; k++)
        if ((cams[k].all_map != nullptr) != planes) return CGX_EINVAL;     // one record form per call
    int k0 = 0;
    while (k0 < n_cameras) {
        // as many consecutive cameras per launch as the parameter block holds
        ExchangeBatch b;
        memset(&b, 0, sizeof(b));
        int n = 0, entries = 0, max_blocks = 0;
        while (k0 + n < n_cameras && n < MAX_XCAMS) {
            const cgx_exchange_camera& c = cams[k0 + n];
            if (c.P < 0 || c.W <= 0 || c.H <= 0 || c.ws <= 0 || c.ws > MAX_WS || !c.dst) return CGX_EINVAL;
            if (entries + (int)c.ws > MAX_XENTRIES) break;
            ExchangeCamera& x = b.cam[n];
            x.P = (int)c.P;
            x.ws = (int)c.ws;
            x.gx = ((int)c.W + CGX_BLOCK_X - 1) / CGX_BLOCK_X;
            x.gy = ((int)c.H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y;
            x.nblocks = (x.P + PACK_TILE - 1) / PACK_TILE;
            x.avoid = c.avoid_pixel_all2all != 0;
            x.entry0 = entries;
            if (x.P > 0) {
                if (!c.means2D || !c.rgb || !c.conic_opacity || !c.radii || !c.depths || !c.tile_bounds || !c.workspace)
                    return CGX_EINVAL;
                if (!planes && (!c.means3D || !c.scales || !c.rotations || !aligned16(c.rotations))) return CGX_EINVAL;
                if (send_index && !c.send_row_offset) return CGX_EINVAL;
                if (((uintptr_t)c.means2D & 7) || !aligned16(c.conic_opacity)) return CGX_EINVAL;
                if ((size_t)c.workspace_bytes < cgx_local2j_workspace_bytes(x.P, x.ws)) return CGX_ENOMEM;
            }
            x.means2D = (const float2*)c.means2D;
            x.rgb = c.rgb;
            x.conic_opacity = (const float4*)c.conic_opacity;
            x.means3D = planes ? c.all_map : c.means3D;
            x.scales = c.scales;
            x.rotations = (const float4*)c.rotations;
            x.radii = c.radii;
            x.depths = c.depths;
            x.bounds = c.tile_bounds;
            x.block_prefix = (const uint32_t*)c.workspace;
            for (int j = 0; j < x.ws; j++) {
                const cgx_peer_camera_dst& d = c.dst[j];
                if (x.P > 0) {
                    if (!d.means2D || !d.rgb || !d.conic_opacity || !d.radii || !d.depths || d.first_row < 0)
                        return CGX_EINVAL;
                    if (planes ? !d.all_map : (!d.means3D || !d.scales || !d.rotations || !aligned16(d.rotations)))
                        return CGX_EINVAL;
                    if (((uintptr_t)d.means2D & 7) || !aligned16(d.conic_opacity)) return CGX_EINVAL;
                }
                b.dst[entries + j] = PeerCameraDst{d.means2D, d.rgb, d.conic_opacity, d.means3D, d.scales,
                                                   d.rotations, d.radii, d.depths, (long long)d.first_row, d.all_map};
                b.local_row[entries + j] = c.send_row_offset ? (long long)c.send_row_offset[j] : 0;
            }
            entries += x.ws;
            if (x.nblocks > max_blocks) max_blocks = x.nblocks;
            n++;
        }
        if (n == 0) return CGX_EINVAL;     // one camera with more ranks than a launch can describe
        if (max_blocks > 0) {
            if (planes)
                local2j_pack_p2p_batched_kernel<true><<<dim3((unsigned)max_blocks, (unsigned)n), PACK_TILE, 0,
                                                        (cudaStream_t)stream>>>(b, send_index);
            else
                local2j_pack_p2p_batched_kernel<false><<<dim3((unsigned)max_blocks, (unsigned)n), PACK_TILE, 0,
                                                         (cudaStream_t)stream>>>(b, send_index);
            const int st = check_launch();
            if (st != CGX_OK) return st;
        }
        k0 += n;
    }
    return CGX_OK;
}

extern "C" int cgx_pack_grad_rows_to(int n_segments, float* const* seg_rows, const int64_t* seg_count, int ncols,
                                     int first_segment, const float* d_means2D, const float* d_rgb,
                                     const float* d_conic_opacity, const float* d_means3D, const float* d_scales,
                                     const float* d_rotations, void* stream)
{
    if (n_segments < 0 || n_segments > MAX_WS || (ncols != 9 && ncols != 14 && ncols != 19)) return CGX_EINVAL;
    if (first_segment < 0 || (n_segments > 0 && first_segment >= n_segments)) return CGX_EINVAL;
    if (n_segments == 0) return CGX_OK;
    if (!seg_rows || !seg_count) return CGX_EINVAL;
    GradSegments sg;
    sg.n = n_segments;
    sg.prefix[0] = 0;
    for (int r = 0; r < n_segments; r++) {
        if (seg_count[r] < 0 || (seg_count[r] > 0 && !seg_rows[r])) return CGX_EINVAL;
        sg.rows[r] = seg_rows[r];
        sg.prefix[r + 1] = sg.prefix[r] + seg_count[r];
    }
    const long long n = sg.prefix[n_segments];
    if (n == 0) return CGX_OK;
    sg.first_row = sg.prefix[first_segment] < n ? sg.prefix[first_segment] : 0;
    if (ncols == 9)
        pack_grad_rows_to_kernel<9><<<(unsigned)((n * 9 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            sg, d_means2D, d_rgb, d_conic_opacity, d_means3D, d_scales, d_rotations);
    else if (ncols == 14)
        pack_grad_rows_to_kernel<14><<<(unsigned)((n * 14 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            sg, d_means2D, d_rgb, d_conic_opacity, d_means3D, nullptr, nullptr);
    else
        pack_grad_rows_to_kernel<19><<<(unsigned)((n * 19 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            sg, d_means2D, d_rgb, d_conic_opacity, d_means3D, d_scales, d_rotations);
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Sorting without any caller-provided or freshly allocated scratch.
//
// Some hosts of this library are not allowed to allocate device memory at the point where they sort: a
// renderer embedded in an engine whose memory budget is fixed at start-up, a plugin that runs after its host
// has frozen the CUDA memory pools, or a service that must not touch the allocator on its latency path because
// cudaMalloc can synchronise the whole device.  For them the digit tables of the radix sort live in the fixed
// array below, which is part of the loaded module: every GPU that loads the library carries these bytes until
// the process exits, so the ceiling is kept modest.
#define CGX_SORT_STATIC_MAX_PAIRS (1 << 22)   // 4,194,304 (key, value) pairs
namespace cgx {
constexpr size_t SORT_STATIC_BYTES =
    ((size_t)(CGX_SORT_STATIC_MAX_PAIRS / SORT_TILE) * RADIX * sizeof(uint32_t) + 255) / 256 * 256 + 1024;
static __device__ __align__(256) unsigned char g_sort_static_scratch[SORT_STATIC_BYTES];
}  // namespace cgx

#include <mutex>

// Device address of the fixed scratch, looked up once per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, so the address is asked for explicitly.
static int sort_static_scratch_ptr(void** out)
{
    constexpr int MAX_DEVICES = 64;
    static std::mutex mu;
    static void* ptrs[MAX_DEVICES] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    if (dev < 0 || dev >= MAX_DEVICES) return CGX_EINVAL;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, cgx::g_sort_static_scratch);
        if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return CGX_OK;
}

extern "C" int64_t cgx_sort_pairs_static_max(void) { return CGX_SORT_STATIC_MAX_PAIRS; }

extern "C" int cgx_sort_pairs_static(int64_t n, int end_bit, uint64_t* keys_in, uint32_t* values_in,
                                     uint64_t* keys_out, uint32_t* values_out, void* stream)
{
    if (n > CGX_SORT_STATIC_MAX_PAIRS) {
        cgx::set_error_text("cgx_sort_pairs_static: n exceeds the fixed scratch (at most 4194304 pairs); "
                            "use cgx_sort_pairs with a caller-provided workspace");
        return CGX_ENOMEM;
    }
    void* scratch = nullptr;
    const int st = sort_static_scratch_ptr(&scratch);
    if (st != CGX_OK) return st;
    // the fixed scratch is sized for the three-kernel passes (digit tables only)
    return sort_pairs_into_out(g_sort_variant == 2 ? -1 : g_sort_variant, n, end_bit, keys_in, values_in, keys_out,
                               values_out, scratch, cgx::SORT_STATIC_BYTES, stream);
}

extern "C" int cgx_unpack_grad_add_cols(int n_ranges, const int64_t* range_start, const int64_t* range_stop, int ncols,
                                        const float* grad_rows, const int32_t* send_index, float* d_means2D,
                                        float* d_rgb, float* d_conic_opacity, float* d_means3D, float* d_scales,
                                        float* d_rotations, void* stream)
{
    if (n_ranges < 0 || n_ranges > MAX_WS || (ncols != 9 && ncols != 14 && ncols != 19)) return CGX_EINVAL;
    if (n_ranges == 0) return CGX_OK;
    if (!range_start || !range_stop) return CGX_EINVAL;
    RowRanges rr;
    rr.n = n_ranges;
    rr.prefix[0] = 0;
    for (int r = 0; r < n_ranges; r++) {
        if (range_stop[r] < range_start[r] || range_start[r] < 0) return CGX_EINVAL;
        rr.start[r] = range_start[r];
        rr.prefix[r + 1] = rr.prefix[r] + (range_stop[r] - range_start[r]);
    }
    const long long total = rr.prefix[n_ranges] * ncols;
    if (total == 0) return CGX_OK;
    if (!grad_rows || !send_index || !d_means2D || !d_conic_opacity) return CGX_EINVAL;
    if (ncols == 9)
        unpack_grad_add_cols_kernel<9><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            rr, grad_rows, send_index, d_means2D, d_rgb, d_conic_opacity, d_means3D, d_scales, d_rotations);
    else if (ncols == 14)
        unpack_grad_add_cols_kernel<14><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            rr, grad_rows, send_index, d_means2D, d_rgb, d_conic_opacity, d_means3D, nullptr, nullptr);
    else
        unpack_grad_add_cols_kernel<19><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            rr, grad_rows, send_index, d_means2D, d_rgb, d_conic_opacity, d_means3D, d_scales, d_rotations);
    return check_launch();
}
