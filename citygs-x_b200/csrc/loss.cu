// Strip loss: masked L1 and masked 11x11 Gaussian-window SSIM of a rendered strip against its ground truth, with the
// gradient towards the rendered strip.  Restates, as two fused kernels, what the reference computes with five grouped
// convolutions and a dozen element-wise tensor ops per strip per step (utils/loss_utils.py:88-132
// pixelwise_l1_with_mask / pixelwise_ssim_with_mask, driven by gaussian_renderer/loss_distribution.py:2835-2885); the
// time of this stage also feeds the tile-row balancer (workload_division.py, `forward_loss_time`).
//
// Forward: one CTA per 16x16 pixel block per channel stages the 26x26 neighbourhood of both images in shared memory,
// runs the separable 11-tap window (zero padding outside the strip, like conv2d(padding=5)) over x, y, x^2, y^2, xy,
// forms the SSIM value, accumulates the two masked sums, and stores the three partial derivatives of the SSIM value
// with respect to the window moments E[x], E[x^2], E[xy] (already masked) for the backward.
// Backward: dL/dx(q) = w_l1 * mask(q) * sign(x(q) - y(q))
//                     + w_ssim * sum_p win(p - q) * [D_mu(p) + 2 x(q) D_xx(p) + y(q) D_xy(p)],
// i.e. the same separable window over the three stored maps.
#include <cmath>

#include "cgx_common.cuh"

namespace cgx {

constexpr int LB = 16;            // pixels per CTA side
constexpr int LR = 5;             // window radius (11 taps)
constexpr int LT = LB + 2 * LR;   // staged side

// gauss(11, sigma 1.5) normalised, in float as the reference builds it (utils/loss_utils.py:27-35)
__constant__ float c_win[11];
static float h_win[11];
static bool h_win_ready[64] = {false};

// Sum over the 256 threads of the CTA (tid = linear thread index); the result is valid in thread 0.
__device__ __forceinline__ float block_sum_256(float v, int tid, float* s_red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = tid & 31, warp = tid >> 5;
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.f;
    if (tid < 8) t = s_red[tid];
    if (warp == 0) {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    }
    return t;
}

__global__ void __launch_bounds__(LB * LB)
strip_loss_fwd_kernel(int H, int W, const float* __restrict__ img, const float* __restrict__ gt,
                      const uint8_t* __restrict__ mask, double* __restrict__ sums, float* __restrict__ d_mu,
                      float* __restrict__ d_xx, float* __restrict__ d_xy)
{
    __shared__ float s_x[LT][LT + 1];
    __shared__ float s_y[LT][LT + 1];
    __shared__ float s_h[5][LT][LB + 1];   // horizontal pass of x, y, xx, yy, xy
    __shared__ float s_red[8];

    const int c = blockIdx.z;
    const size_t plane = (size_t)c * H * W;
    const int x0 = blockIdx.x * LB - LR, y0 = blockIdx.y * LB - LR;
    const int tid = threadIdx.y * LB + threadIdx.x;
    for (int e = tid; e < LT * LT; e += LB * LB) {
        const int r = e / LT, q = e - r * LT;
        const int yy = y0 + r, xx = x0 + q;
        float a = 0.f, b = 0.f;
        if (yy >= 0 && yy < H && xx >= 0 && xx < W) {
            a = img[plane + (size_t)yy * W + xx];
            b = gt[plane + (size_t)yy * W + xx];
        }
        s_x[r][q] = a;
        s_y[r][q] = b;
    }
    __syncthreads();
    for (int e = tid; e < LT * LB; e += LB * LB) {
        const int r = e / LB, q = e - r * LB;
        float mx = 0.f, my = 0.f, mxx = 0.f, myy = 0.f, mxy = 0.f;
#pragma unroll
        for (int k = 0; k < 11; k++) {
            const float w = c_win[k], a = s_x[r][q + k], b = s_y[r][q + k];
            mx += w * a;
            my += w * b;
            mxx += w * a * a;
            myy += w * b * b;
            mxy += w * a * b;
        }
        s_h[0][r][q] = mx; s_h[1][r][q] = my; s_h[2][r][q] = mxx; s_h[3][r][q] = myy; s_h[4][r][q] = mxy;
    }
    __syncthreads();
    const int px = blockIdx.x * LB + threadIdx.x, py = blockIdx.y * LB + threadIdx.y;
    float l1 = 0.f, ss = 0.f;
    if (px < W && py < H) {
        float mu1 = 0.f, mu2 = 0.f, exx = 0.f, eyy = 0.f, exy = 0.f;
#pragma unroll
        for (int k = 0; k < 11; k++) {
            const float w = c_win[k];
            mu1 += w * s_h[0][threadIdx.y + k][threadIdx.x];
            mu2 += w * s_h[1][threadIdx.y + k][threadIdx.x];
            exx += w * s_h[2][threadIdx.y + k][threadIdx.x];
            eyy += w * s_h[3][threadIdx.y + k][threadIdx.x];
            exy += w * s_h[4][threadIdx.y + k][threadIdx.x];
        }
        const float C1 = 0.01f * 0.01f, C2 = 0.03f * 0.03f;
        const float s1 = exx - mu1 * mu1, s2 = eyy - mu2 * mu2, s12 = exy - mu1 * mu2;
        const float A1 = 2.f * mu1 * mu2 + C1, A2 = 2.f * s12 + C2;
        const float B1 = mu1 * mu1 + mu2 * mu2 + C1, B2 = s1 + s2 + C2;
        const float inv = 1.f / (B1 * B2);
        const float val = A1 * A2 * inv;
        const float m = mask ? (mask[(size_t)py * W + px] ? 1.f : 0.f) : 1.f;
        const size_t o = plane + (size_t)py * W + px;
        if (d_mu) {
            // derivatives with respect to the window moments, E[x^2] and E[xy] held fixed for the first one
            const float dnum = 2.f * mu2 * A2 - 2.f * mu2 * A1;              // d(A1 A2)/d mu1
            const float dden = 2.f * mu1 * B2 - 2.f * mu1 * B1;              // d(B1 B2)/d mu1
            d_mu[o] = m * (dnum - val * dden) * inv;
            d_xx[o] = m * (-val / B2);
            d_xy[o] = m * (2.f * A1 * inv);
        }
        const float a = s_x[threadIdx.y + LR][threadIdx.x + LR], b = s_y[threadIdx.y + LR][threadIdx.x + LR];
        l1 = m * fabsf(a - b);
        ss = m * val;
    }
    const float t1 = block_sum_256(l1, tid, s_red);
    const float t2 = block_sum_256(ss, tid, s_red);
    if (tid == 0) {      // thousands of CTA partial sums: accumulated in double so that their order does not matter
        atomicAdd(sums, (double)t1);
        atomicAdd(sums + 1, (double)t2);
    }
}

__global__ void __launch_bounds__(LB * LB)
strip_loss_bwd_kernel(int H, int W, const float* __restrict__ img, const float* __restrict__ gt,
                      const uint8_t* __restrict__ mask, const float* __restrict__ weights,
                      const float* __restrict__ d_mu, const float* __restrict__ d_xx, const float* __restrict__ d_xy,
                      float* __restrict__ dL_dimg)
{
    __shared__ float s_m[3][LT][LT + 1];
    __shared__ float s_h[3][LT][LB + 1];

    const int c = blockIdx.z;
    const size_t plane = (size_t)c * H * W;
    const int x0 = blockIdx.x * LB - LR, y0 = blockIdx.y * LB - LR;
    const int tid = threadIdx.y * LB + threadIdx.x;
    for (int e = tid; e < LT * LT; e += LB * LB) {
        const int r = e / LT, q = e - r * LT;
        const int yy = y0 + r, xx = x0 + q;
        float a = 0.f, b = 0.f, d = 0.f;
        if (yy >= 0 && yy < H && xx >= 0 && xx < W) {
            const size_t o = plane + (size_t)yy * W + xx;
            a = d_mu[o];
            b = d_xx[o];
            d = d_xy[o];
        }
        s_m[0][r][q] = a;
        s_m[1][r][q] = b;
        s_m[2][r][q] = d;
    }
    __syncthreads();
    for (int e = tid; e < LT * LB; e += LB * LB) {
        const int r = e / LB, q = e - r * LB;
        float a = 0.f, b = 0.f, d = 0.f;
#pragma unroll
        for (int k = 0; k < 11; k++) {
            const float w = c_win[k];
            a += w * s_m[0][r][q + k];
            b += w * s_m[1][r][q + k];
            d += w * s_m[2][r][q + k];
        }
        s_h[0][r][q] = a; s_h[1][r][q] = b; s_h[2][r][q] = d;
    }
    __syncthreads();
    const int px = blockIdx.x * LB + threadIdx.x, py = blockIdx.y * LB + threadIdx.y;
    if (px >= W || py >= H) return;
    float a = 0.f, b = 0.f, d = 0.f;
#pragma unroll
    for (int k = 0; k < 11; k++) {
        const float w = c_win[k];
        a += w * s_h[0][threadIdx.y + k][threadIdx.x];
        b += w * s_h[1][threadIdx.y + k][threadIdx.x];
        d += w * s_h[2][threadIdx.y + k][threadIdx.x];
    }
    const size_t o = plane + (size_t)py * W + px;
    const float x = img[o], y = gt[o];
    const float m = mask ? (mask[(size_t)py * W + px] ? 1.f : 0.f) : 1.f;
    const float diff = x - y;
    const float sgn = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
    dL_dimg[o] = weights[0] * m * sgn + weights[1] * (a + 2.f * x * b + y * d);
}

// ---------------------------------------------------------------------------------------------------------------
// Normal image from a depth image (render_normal, gaussian_renderer/__init__.py:1311-1323 with scale = 1 and no
// offsets -> normal_from_depth_image / depth_pcd2normal, utils/graphics_utils.py:87-152): camera-space points
// p(x,y) = z * ((x - cx)/fx, (y - cy)/fy, 1), normal = normalize((p_right - p_left) x (p_top - p_bottom)) with
// bottom = row + 1, top = row - 1, zero on the one-pixel border.
struct Pinhole {
    float fx, fy, cx, cy;
};

__device__ __forceinline__ float3 depth_point(const float* __restrict__ depth, int W, int x, int y, const Pinhole k)
{
    const float z = depth[(size_t)y * W + x];
    return make_float3(z * (((float)x - k.cx) / k.fx), z * (((float)y - k.cy) / k.fy), z);
}

__device__ __forceinline__ float3 cross3(const float3 a, const float3 b)
{
    return make_float3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}

// a = right - left, b = top - bottom, c = a x b of the interior pixel (x, y)
__device__ __forceinline__ void normal_frame(const float* __restrict__ depth, int W, int x, int y, const Pinhole k,
                                             float3& a, float3& b, float3& c)
{
    const float3 pr = depth_point(depth, W, x + 1, y, k), pl = depth_point(depth, W, x - 1, y, k);
    const float3 pt = depth_point(depth, W, x, y - 1, k), pb = depth_point(depth, W, x, y + 1, k);
    a = make_float3(pr.x - pl.x, pr.y - pl.y, pr.z - pl.z);
    b = make_float3(pt.x - pb.x, pt.y - pb.y, pt.z - pb.z);
    c = cross3(a, b);
}

__global__ void __launch_bounds__(256)
depth_normal_fwd_kernel(int H, int W, Pinhole k, const float* __restrict__ depth, float* __restrict__ normal)
{
    const int x = blockIdx.x * 32 + (threadIdx.x & 31), y = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (x >= W || y >= H) return;
    float3 n = make_float3(0.f, 0.f, 0.f);
    if (x > 0 && x < W - 1 && y > 0 && y < H - 1) {
        float3 a, b, c;
        normal_frame(depth, W, x, y, k, a, b, c);
        const float len = fmaxf(sqrtf(c.x * c.x + c.y * c.y + c.z * c.z), 1e-12f);
        n = make_float3(c.x / len, c.y / len, c.z / len);
    }
    const size_t HW = (size_t)H * W, o = (size_t)y * W + x;
    normal[o] = n.x;
    normal[HW + o] = n.y;
    normal[2 * HW + o] = n.z;
}

// Cotangent of the cross product c of interior pixel (x, y) given the cotangent g of its unit normal.
__device__ __forceinline__ bool normal_cotangent(const float* __restrict__ depth, const float* __restrict__ g, int H,
                                                 int W, int x, int y, const Pinhole k, float3& a, float3& b,
                                                 float3& gc)
{
    if (x <= 0 || x >= W - 1 || y <= 0 || y >= H - 1) return false;
    float3 c;
    normal_frame(depth, W, x, y, k, a, b, c);
    const float len = sqrtf(c.x * c.x + c.y * c.y + c.z * c.z);
    if (!(len > 1e-12f)) return false;            // clamped norm: the direction carries no gradient
    const size_t HW = (size_t)H * W, o = (size_t)y * W + x;
    const float3 gn = make_float3(g[o], g[HW + o], g[2 * HW + o]);
    const float3 n = make_float3(c.x / len, c.y / len, c.z / len);
    const float d = n.x * gn.x + n.y * gn.y + n.z * gn.z;
    gc = make_float3((gn.x - n.x * d) / len, (gn.y - n.y * d) / len, (gn.z - n.z * d) / len);
    return true;
}

// Gather form: a depth pixel is the right / left / top / bottom point of four neighbouring normals.
__global__ void __launch_bounds__(256)
depth_normal_bwd_kernel(int H, int W, Pinhole k, const float* __restrict__ depth, const float* __restrict__ g,
                        float* __restrict__ dL_ddepth)
{
    const int x = blockIdx.x * 32 + (threadIdx.x & 31), y = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (x >= W || y >= H) return;
    float3 gp = make_float3(0.f, 0.f, 0.f);       // cotangent of this pixel's camera-space point
    float3 a, b, gc;
    // c = a x b:  dL/da = b x gc,  dL/db = gc x a
    if (normal_cotangent(depth, g, H, W, x - 1, y, k, a, b, gc)) {        // right point of (x-1, y): +dL/da
        const float3 t = cross3(b, gc);
        gp.x += t.x; gp.y += t.y; gp.z += t.z;
    }
    if (normal_cotangent(depth, g, H, W, x + 1, y, k, a, b, gc)) {        // left point of (x+1, y): -dL/da
        const float3 t = cross3(b, gc);
        gp.x -= t.x; gp.y -= t.y; gp.z -= t.z;
    }
    if (normal_cotangent(depth, g, H, W, x, y + 1, k, a, b, gc)) {        // top point of (x, y+1): +dL/db
        const float3 t = cross3(gc, a);
        gp.x += t.x; gp.y += t.y; gp.z += t.z;
    }
    if (normal_cotangent(depth, g, H, W, x, y - 1, k, a, b, gc)) {        // bottom point of (x, y-1): -dL/db
        const float3 t = cross3(gc, a);
        gp.x -= t.x; gp.y -= t.y; gp.z -= t.z;
    }
    dL_ddepth[(size_t)y * W + x] = gp.x * (((float)x - k.cx) / k.fx) + gp.y * (((float)y - k.cy) / k.fy) + gp.z;
}

static int upload_window()
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return CGX_ECUDA;
    }
    if (dev < 0 || dev >= 64) return CGX_EINVAL;
    if (h_win_ready[dev]) return CGX_OK;
    float g[11], sum = 0.f;
    for (int x = 0; x < 11; x++) {
        g[x] = (float)exp(-(double)((x - 5) * (x - 5)) / (2.0 * 1.5 * 1.5));   // stored to float first, as torch.Tensor does
        sum += g[x];                                                          // float sum, ascending
    }
    for (int x = 0; x < 11; x++) h_win[x] = g[x] / sum;
    e = cudaMemcpyToSymbol(c_win, h_win, sizeof(h_win));
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return CGX_ECUDA;
    }
    h_win_ready[dev] = true;
    return CGX_OK;
}

}  // namespace cgx

using namespace cgx;

extern "C" int cgx_strip_loss_fwd(int C, int H, int W, const float* img, const float* gt, const uint8_t* mask,
                                  double* sums, float* d_mu, float* d_xx, float* d_xy, void* stream)
{
    if (C <= 0 || H <= 0 || W <= 0 || !img || !gt || !sums) return CGX_EINVAL;
    if ((d_mu != nullptr) != (d_xx != nullptr) || (d_mu != nullptr) != (d_xy != nullptr)) return CGX_EINVAL;
    int st = upload_window();
    if (st != CGX_OK) return st;
    cudaError_t e = cudaMemsetAsync(sums, 0, 2 * sizeof(double), (cudaStream_t)stream);
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return CGX_ECUDA;
    }
    dim3 grid((W + LB - 1) / LB, (H + LB - 1) / LB, C), block(LB, LB);
    strip_loss_fwd_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(H, W, img, gt, mask, sums, d_mu, d_xx, d_xy);
    return check_launch();
}

extern "C" int cgx_strip_loss_bwd(int C, int H, int W, const float* img, const float* gt, const uint8_t* mask,
                                  const float* weights, const float* d_mu, const float* d_xx, const float* d_xy,
                                  float* dL_dimg, void* stream)
{
    if (C <= 0 || H <= 0 || W <= 0 || !img || !gt || !weights || !d_mu || !d_xx || !d_xy || !dL_dimg)
        return CGX_EINVAL;
    int st = upload_window();
    if (st != CGX_OK) return st;
    dim3 grid((W + LB - 1) / LB, (H + LB - 1) / LB, C), block(LB, LB);
    strip_loss_bwd_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(H, W, img, gt, mask, weights, d_mu, d_xx, d_xy,
                                                                    dL_dimg);
    return check_launch();
}

extern "C" int cgx_depth_normal_fwd(int H, int W, float fx, float fy, float cx, float cy, const float* depth,
                                    float* normal, void* stream)
{
    if (H <= 0 || W <= 0 || !depth || !normal || fx == 0.f || fy == 0.f) return CGX_EINVAL;
    dim3 grid((W + 31) / 32, (H + 7) / 8);
    depth_normal_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(H, W, Pinhole{fx, fy, cx, cy}, depth, normal);
    return check_launch();
}

extern "C" int cgx_depth_normal_bwd(int H, int W, float fx, float fy, float cx, float cy, const float* depth,
                                    const float* dL_dnormal, float* dL_ddepth, void* stream)
{
    if (H <= 0 || W <= 0 || !depth || !dL_dnormal || !dL_ddepth || fx == 0.f || fy == 0.f) return CGX_EINVAL;
    dim3 grid((W + 31) / 32, (H + 7) / 8);
    depth_normal_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(H, W, Pinhole{fx, fy, cx, cy}, depth, dL_dnormal,
                                                                    dL_ddepth);
    return check_launch();
}
