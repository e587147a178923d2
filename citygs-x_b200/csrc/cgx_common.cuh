// Shared device helpers for the cgx_raster kernels (sm_100a).
//
// The float expressions in this file are written in the same operand order as the
// reference rasterizer's device code so that nvcc's default FMA contraction produces the
// same bits: integer outputs (radii, tile rectangles, sort keys) depend on them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/cgx_raster.h"
#include "../../include/cgx_raster_testing.h"

#define CGX_BLOCK_X 16
#define CGX_BLOCK_Y 16
#define CGX_BLOCK_SIZE 256
#define CGX_NCH 3
#define CGX_NMAP 5

namespace cgx {

void set_cuda_error(cudaError_t e);
void set_error_text(const char* text);  // free-form text behind cgx_last_cuda_error()
// Checks for a launch error; `launched` = number of kernels the entry point just queued (bookkeeping for
// cgx_launch_count()).
int check_launch(int launched = 1);
// A few 32-bit words from device memory to page-locked host memory by a one-CTA kernel (stores through the host
// mapping), so that the read-back does not queue behind bulk copies on the device-to-host copy engine.
int post_words(const void* src_dev, void* dst_host_pinned, int n_words, cudaStream_t st);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Column-major 3x3 (m[c][r]); product order matches the usual column-major definition
// r[c][row] = a[0][row]*b[c][0] + a[1][row]*b[c][1] + a[2][row]*b[c][2], summed left to right.
struct Mat3 {
    float m[3][3];
};

__device__ __forceinline__ Mat3 mul(const Mat3& a, const Mat3& b)
{
    Mat3 r;
#pragma unroll
    for (int c = 0; c < 3; c++)
#pragma unroll
        for (int row = 0; row < 3; row++)
            r.m[c][row] = a.m[0][row] * b.m[c][0] + a.m[1][row] * b.m[c][1] + a.m[2][row] * b.m[c][2];
    return r;
}

__device__ __forceinline__ Mat3 transpose(const Mat3& a)
{
    Mat3 r;
#pragma unroll
    for (int c = 0; c < 3; c++)
#pragma unroll
        for (int row = 0; row < 3; row++) r.m[c][row] = a.m[row][c];
    return r;
}

__device__ __forceinline__ float ndc2pix(float v, int S) { return ((v + 1.0) * S - 1.0) * 0.5; }

// Tile rectangle of a splat (RAST/cuda_rasterizer/auxiliary.h:66-76).
__device__ __forceinline__ void get_rect(const float2 p, int max_radius, uint2& rect_min, uint2& rect_max, int gx, int gy)
{
    rect_min = {(unsigned)min(gx, max((int)0, (int)((p.x - max_radius) / CGX_BLOCK_X))),
                (unsigned)min(gy, max((int)0, (int)((p.y - max_radius) / CGX_BLOCK_Y)))};
    rect_max = {(unsigned)min(gx, max((int)0, (int)((p.x + max_radius + CGX_BLOCK_X - 1) / CGX_BLOCK_X))),
                (unsigned)min(gy, max((int)0, (int)((p.y + max_radius + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y)))};
}

__device__ __forceinline__ float3 transform_point_4x3(const float3& p, const float* matrix)
{
    float3 transformed = {
        matrix[0] * p.x + matrix[4] * p.y + matrix[8] * p.z + matrix[12],
        matrix[1] * p.x + matrix[5] * p.y + matrix[9] * p.z + matrix[13],
        matrix[2] * p.x + matrix[6] * p.y + matrix[10] * p.z + matrix[14],
    };
    return transformed;
}

__device__ __forceinline__ float4 transform_point_4x4(const float3& p, const float* matrix)
{
    float4 transformed = {matrix[0] * p.x + matrix[4] * p.y + matrix[8] * p.z + matrix[12],
                          matrix[1] * p.x + matrix[5] * p.y + matrix[9] * p.z + matrix[13],
                          matrix[2] * p.x + matrix[6] * p.y + matrix[10] * p.z + matrix[14],
                          matrix[3] * p.x + matrix[7] * p.y + matrix[11] * p.z + matrix[15]};
    return transformed;
}

__device__ __forceinline__ float3 transform_vec_4x3_transpose(const float3& p, const float* matrix)
{
    float3 transformed = {
        matrix[0] * p.x + matrix[1] * p.y + matrix[2] * p.z,
        matrix[4] * p.x + matrix[5] * p.y + matrix[6] * p.z,
        matrix[8] * p.x + matrix[9] * p.y + matrix[10] * p.z,
    };
    return transformed;
}

// Cooperative, vectorised copy of `count` consecutive AoS rows of WIDTH floats between global and shared
// memory.  `g` points at the first row of the block.  When vec_ok (16-byte aligned base) the bulk moves as
// float4; the ragged tail and unaligned arrays move as scalars.
template <int WIDTH>
__device__ __forceinline__ void block_load_rows(const float* __restrict__ g, float* s, int count, bool vec_ok)
{
    const int nfl = count * WIDTH;
    if (vec_ok) {
        const int nv = nfl >> 2;
        const float4* g4 = reinterpret_cast<const float4*>(g);
        float4* s4 = reinterpret_cast<float4*>(s);
        for (int i = threadIdx.x; i < nv; i += blockDim.x) s4[i] = __ldg(g4 + i);
        for (int i = (nv << 2) + threadIdx.x; i < nfl; i += blockDim.x) s[i] = __ldg(g + i);
    } else {
        for (int i = threadIdx.x; i < nfl; i += blockDim.x) s[i] = __ldg(g + i);
    }
}

template <int WIDTH>
__device__ __forceinline__ void block_store_rows(float* __restrict__ g, const float* s, int count, bool vec_ok)
{
    const int nfl = count * WIDTH;
    if (vec_ok) {
        const int nv = nfl >> 2;
        float4* g4 = reinterpret_cast<float4*>(g);
        const float4* s4 = reinterpret_cast<const float4*>(s);
        for (int i = threadIdx.x; i < nv; i += blockDim.x) g4[i] = s4[i];
        for (int i = (nv << 2) + threadIdx.x; i < nfl; i += blockDim.x) g[i] = s[i];
    } else {
        for (int i = threadIdx.x; i < nfl; i += blockDim.x) g[i] = s[i];
    }
}

}  // namespace cgx
