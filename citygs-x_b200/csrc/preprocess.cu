// Per-Gaussian stages: projection / EWA covariance / radius (forward), the anchor visibility
// filter, the frustum mark, the optional SH->RGB stage and the fused preprocess backward.
//
// Memory plan (HBM-bound kernels): one thread per Gaussian, 256 Gaussians per CTA.  The AoS
// inputs ((P,3),(P,3),(P,4)) are pulled in as 128-bit loads by the whole CTA into shared
// memory and read back with conflict-free strides (3 and 4 words); the (P,6) covariance output
// takes the same route in reverse, so every global transaction is a full 16-byte vector.
// Outputs are written for every Gaussian (zeros for culled ones), so callers need no memsets.
#include "cgx_common.cuh"

namespace cgx {

// Scale + (unnormalised) quaternion -> upper triangle of the world-space covariance.
__device__ __forceinline__ void compute_cov3d(const float3 scale, float mod, const float4 rot, float* cov3D)
{
    Mat3 S;
#pragma unroll
    for (int c = 0; c < 3; c++)
#pragma unroll
        for (int r = 0; r < 3; r++) S.m[c][r] = 0.0f;
    S.m[0][0] = mod * scale.x;
    S.m[1][1] = mod * scale.y;
    S.m[2][2] = mod * scale.z;

    float r = rot.x;
    float x = rot.y;
    float y = rot.z;
    float z = rot.w;

    Mat3 R;
    R.m[0][0] = 1.f - 2.f * (y * y + z * z); R.m[0][1] = 2.f * (x * y - r * z); R.m[0][2] = 2.f * (x * z + r * y);
    R.m[1][0] = 2.f * (x * y + r * z); R.m[1][1] = 1.f - 2.f * (x * x + z * z); R.m[1][2] = 2.f * (y * z - r * x);
    R.m[2][0] = 2.f * (x * z - r * y); R.m[2][1] = 2.f * (y * z + r * x); R.m[2][2] = 1.f - 2.f * (x * x + y * y);

    Mat3 M = mul(S, R);
    Mat3 Sigma = mul(transpose(M), M);

    cov3D[0] = Sigma.m[0][0];
    cov3D[1] = Sigma.m[0][1];
    cov3D[2] = Sigma.m[0][2];
    cov3D[3] = Sigma.m[1][1];
    cov3D[4] = Sigma.m[1][2];
    cov3D[5] = Sigma.m[2][2];
}

// EWA projection of the 3-D covariance (Zwicker et al. 2002, eq. 29/31) plus the 0.3 px low-pass.
__device__ __forceinline__ float3 compute_cov2d(const float3& mean, float focal_x, float focal_y, float tan_fovx,
                                                float tan_fovy, const float* cov3D, const float* viewmatrix)
{
    float3 t = transform_point_4x3(mean, viewmatrix);

    const float limx = 1.3f * tan_fovx;
    const float limy = 1.3f * tan_fovy;
    const float txtz = t.x / t.z;
    const float tytz = t.y / t.z;
    t.x = min(limx, max(-limx, txtz)) * t.z;
    t.y = min(limy, max(-limy, tytz)) * t.z;

    Mat3 J;
    J.m[0][0] = focal_x / t.z; J.m[0][1] = 0.0f; J.m[0][2] = -(focal_x * t.x) / (t.z * t.z);
    J.m[1][0] = 0.0f; J.m[1][1] = focal_y / t.z; J.m[1][2] = -(focal_y * t.y) / (t.z * t.z);
    J.m[2][0] = 0; J.m[2][1] = 0; J.m[2][2] = 0;

    Mat3 W;
    W.m[0][0] = viewmatrix[0]; W.m[0][1] = viewmatrix[4]; W.m[0][2] = viewmatrix[8];
    W.m[1][0] = viewmatrix[1]; W.m[1][1] = viewmatrix[5]; W.m[1][2] = viewmatrix[9];
    W.m[2][0] = viewmatrix[2]; W.m[2][1] = viewmatrix[6]; W.m[2][2] = viewmatrix[10];

    Mat3 T = mul(W, J);

    Mat3 Vrk;
    Vrk.m[0][0] = cov3D[0]; Vrk.m[0][1] = cov3D[1]; Vrk.m[0][2] = cov3D[2];
    Vrk.m[1][0] = cov3D[1]; Vrk.m[1][1] = cov3D[3]; Vrk.m[1][2] = cov3D[4];
    Vrk.m[2][0] = cov3D[2]; Vrk.m[2][1] = cov3D[4]; Vrk.m[2][2] = cov3D[5];

    Mat3 cov = mul(mul(transpose(T), transpose(Vrk)), T);

    cov.m[0][0] += 0.3f;
    cov.m[1][1] += 0.3f;
    return {float(cov.m[0][0]), float(cov.m[0][1]), float(cov.m[1][1])};
}

template <bool FILTER>
__global__ void __launch_bounds__(CGX_BLOCK_SIZE)
preprocess_fwd_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ scales,
                      const float scale_modifier, const float* __restrict__ rotations,
                      const float* __restrict__ opacities, const float* __restrict__ viewmatrix_g,
                      const float* __restrict__ projmatrix_g, const int W, int H, const float tan_fovx,
                      float tan_fovy, const float focal_x, float focal_y, int* __restrict__ radii,
                      float2* __restrict__ points_xy_image, float* __restrict__ depths,
                      float* __restrict__ cov3Ds, float4* __restrict__ conic_opacity, int vec_mask,
                      const float* __restrict__ cov3D_precomp)
{
    // cov3D_precomp (filter only): six floats per Gaussian given by the caller instead of scales and rotations
    // (cuda_rasterizer/forward.cu:585-595 of the reference)
    __shared__ __align__(16) float s_mean[CGX_BLOCK_SIZE * 3];
    __shared__ __align__(16) float s_scale[CGX_BLOCK_SIZE * 3];
    __shared__ __align__(16) float s_rot[CGX_BLOCK_SIZE * 4];
    __shared__ __align__(16) float s_cov[FILTER ? 4 : CGX_BLOCK_SIZE * 6];
    __shared__ float viewmatrix[16];
    __shared__ float projmatrix[16];

    const int base = blockIdx.x * CGX_BLOCK_SIZE;
    const int count = min(CGX_BLOCK_SIZE, P - base);
    if (threadIdx.x < 16) viewmatrix[threadIdx.x] = viewmatrix_g[threadIdx.x];
    else if (threadIdx.x < 32) projmatrix[threadIdx.x - 16] = projmatrix_g[threadIdx.x - 16];
    block_load_rows<3>(means3D + (size_t)base * 3, s_mean, count, vec_mask & 1);
    if (!(FILTER && cov3D_precomp)) {
        block_load_rows<3>(scales + (size_t)base * 3, s_scale, count, vec_mask & 2);
        block_load_rows<4>(rotations + (size_t)base * 4, s_rot, count, vec_mask & 4);
    }
    __syncthreads();

    const int t = threadIdx.x;
    const int idx = base + t;
    int out_radius = 0;
    float2 out_xy = {0.f, 0.f};
    float out_depth = 0.f;
    float4 out_co = {0.f, 0.f, 0.f, 0.f};
    float cov3D[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};

    if (t < count) {
        do {
            float3 p_orig = {s_mean[3 * t], s_mean[3 * t + 1], s_mean[3 * t + 2]};
            // Near cull in view space: keep z > 0 only (no x/y frustum test).
            float4 p_hom = transform_point_4x4(p_orig, projmatrix);
            float p_w = 1.0f / (p_hom.w + 0.0000001f);
            float3 p_proj = {p_hom.x * p_w, p_hom.y * p_w, p_hom.z * p_w};
            float3 p_view = transform_point_4x3(p_orig, viewmatrix);
            if (p_view.z <= 0.0f) break;

            if (FILTER && cov3D_precomp) {
#pragma unroll
                for (int k = 0; k < 6; k++) cov3D[k] = __ldg(cov3D_precomp + 6 * (size_t)idx + k);
            } else {
                const float3 sc = {s_scale[3 * t], s_scale[3 * t + 1], s_scale[3 * t + 2]};
                const float4 q = {s_rot[4 * t], s_rot[4 * t + 1], s_rot[4 * t + 2], s_rot[4 * t + 3]};
                compute_cov3d(sc, scale_modifier, q, cov3D);
            }

            float3 cov = compute_cov2d(p_orig, focal_x, focal_y, tan_fovx, tan_fovy, cov3D, viewmatrix);

            float det = (cov.x * cov.z - cov.y * cov.y);
            if (det == 0.0f) break;
            float det_inv = 1.f / det;
            float3 conic = {cov.z * det_inv, -cov.y * det_inv, cov.x * det_inv};

            float mid = 0.5f * (cov.x + cov.z);
            float lambda1 = mid + sqrt(max(0.1f, mid * mid - det));
            float lambda2 = mid - sqrt(max(0.1f, mid * mid - det));
            float my_radius = ceil(3.f * sqrt(max(lambda1, lambda2)));
            float2 point_image = {ndc2pix(p_proj.x, W), ndc2pix(p_proj.y, H)};
            uint2 rect_min, rect_max;
            get_rect(point_image, my_radius, rect_min, rect_max, (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X,
                     (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y);
            if ((rect_max.x - rect_min.x) * (rect_max.y - rect_min.y) == 0) break;

            out_depth = p_view.z;
            out_radius = my_radius;
            out_xy = point_image;
            if (!FILTER) out_co = {conic.x, conic.y, conic.z, __ldg(opacities + idx)};
        } while (0);

        radii[idx] = out_radius;
        if (!FILTER) {
            points_xy_image[idx] = out_xy;
            depths[idx] = out_depth;
            conic_opacity[idx] = out_co;
#pragma unroll
            for (int k = 0; k < 6; k++) s_cov[6 * t + k] = cov3D[k];
        }
    }
    if (!FILTER) {
        __syncthreads();
        block_store_rows<6>(cov3Ds + (size_t)base * 6, s_cov, count, vec_mask & 8);
    }
}

__global__ void mark_visible_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ viewmatrix,
                                    uint8_t* __restrict__ present)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= P) return;
    float3 p = {means3D[3 * idx], means3D[3 * idx + 1], means3D[3 * idx + 2]};
    float3 pv = transform_point_4x3(p, viewmatrix);
    present[idx] = pv.z > 0.0f;
}

// Real spherical-harmonic basis constants (degrees 0..3).
__device__ const float SH_C0 = 0.28209479177387814f;
__device__ const float SH_C1 = 0.4886025119029199f;
__device__ const float SH_C2[] = {1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f,
                                  -1.0925484305920792f, 0.5462742152960396f};
__device__ const float SH_C3[] = {-0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f,
                                  -0.4570457994644658f, 1.445305721320277f, -0.5900435899266435f};

// One warp per 32 Gaussians; the (M,3) coefficient block of a Gaussian is contiguous, so the CTA
// streams its 256*M*3 floats through shared memory in 128-bit pieces.
__global__ void __launch_bounds__(128)
sh_to_rgb_kernel(int P, int deg, int M, const float* __restrict__ means3D, const float* __restrict__ campos,
                 const float* __restrict__ shs, float* __restrict__ rgb, uint8_t* __restrict__ clamped, int vec_ok)
{
    extern __shared__ __align__(16) float s_sh[];  // 128 * M * 3 floats
    const int base = blockIdx.x * 128;
    const int count = min(128, P - base);
    {
        const int nfl = count * M * 3;
        const float* g = shs + (size_t)base * M * 3;
        if (vec_ok) {
            const int nv = nfl >> 2;
            for (int i = threadIdx.x; i < nv; i += blockDim.x)
                reinterpret_cast<float4*>(s_sh)[i] = __ldg(reinterpret_cast<const float4*>(g) + i);
            for (int i = (nv << 2) + threadIdx.x; i < nfl; i += blockDim.x) s_sh[i] = __ldg(g + i);
        } else {
            for (int i = threadIdx.x; i < nfl; i += blockDim.x) s_sh[i] = __ldg(g + i);
        }
    }
    __syncthreads();
    const int t = threadIdx.x;
    if (t >= count) return;
    const int idx = base + t;
    float3 pos = {means3D[3 * idx], means3D[3 * idx + 1], means3D[3 * idx + 2]};
    float3 dir = {pos.x - campos[0], pos.y - campos[1], pos.z - campos[2]};
    float len = sqrt(dir.x * dir.x + dir.y * dir.y + dir.z * dir.z);
    dir = {dir.x / len, dir.y / len, dir.z / len};
    // stride M*3 between threads: odd multiples of 3 words are bank-conflict free for M=16 (48 words -> 2-way);
    // accepted, the kernel is bound by the 192 B/Gaussian global read.
    const float* sh = s_sh + (size_t)t * M * 3;
    float x = dir.x, y = dir.y, z = dir.z;
    float res[3];
#pragma unroll
    for (int ch = 0; ch < 3; ch++) {
        float result = SH_C0 * sh[ch];
        if (deg > 0) {
            result = result - SH_C1 * y * sh[3 + ch] + SH_C1 * z * sh[6 + ch] - SH_C1 * x * sh[9 + ch];
            if (deg > 1) {
                float xx = x * x, yy = y * y, zz = z * z;
                float xy = x * y, yz = y * z, xz = x * z;
                result = result + SH_C2[0] * xy * sh[12 + ch] + SH_C2[1] * yz * sh[15 + ch] +
                         SH_C2[2] * (2.0f * zz - xx - yy) * sh[18 + ch] + SH_C2[3] * xz * sh[21 + ch] +
                         SH_C2[4] * (xx - yy) * sh[24 + ch];
                if (deg > 2) {
                    result = result + SH_C3[0] * y * (3.0f * xx - yy) * sh[27 + ch] + SH_C3[1] * xy * z * sh[30 + ch] +
                             SH_C3[2] * y * (4.0f * zz - xx - yy) * sh[33 + ch] +
                             SH_C3[3] * z * (2.0f * zz - 3.0f * xx - 3.0f * yy) * sh[36 + ch] +
                             SH_C3[4] * x * (4.0f * zz - xx - yy) * sh[39 + ch] + SH_C3[5] * z * (xx - yy) * sh[42 + ch] +
                             SH_C3[6] * x * (xx - 3.0f * yy) * sh[45 + ch];
                }
            }
        }
        result += 0.5f;
        res[ch] = result;
    }
#pragma unroll
    for (int ch = 0; ch < 3; ch++) {
        clamped[3 * idx + ch] = (res[ch] < 0);
        rgb[3 * idx + ch] = max(res[ch], 0.0f);
    }
}


// PGSR per-Gaussian plane descriptor for one camera (the tensor code of gaussian_renderer/__init__.py:1501-1518):
// the rotation-matrix column of the smallest scale is the plane normal in world space, flipped to face the camera,
// rotated into camera space; then [normal_cam(3), 1, |normal_cam . p_cam|].  The quaternion is normalised here
// (the caller normalises before converting).  V: 4x4 row-vector view matrix.
__device__ __forceinline__ void plane_fwd(const float3 p, const float3 sc, float4 q, const float* V,
                                          const float3 campos, float* o5)
{
    const float qn = fmaxf(sqrtf(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w), 1e-12f);
    q = {q.x / qn, q.y / qn, q.z / qn, q.w / qn};
    const float r = q.x, x = q.y, y = q.z, z = q.w;
    const float two_s = 2.0f / (r * r + x * x + y * y + z * z);
    int idx = 0;
    float smin = sc.x;
    if (sc.y < smin) { smin = sc.y; idx = 1; }
    if (sc.z < smin) { smin = sc.z; idx = 2; }
    float3 n;
    if (idx == 0) n = {1.f - two_s * (y * y + z * z), two_s * (x * y + z * r), two_s * (x * z - y * r)};
    else if (idx == 1) n = {two_s * (x * y - z * r), 1.f - two_s * (x * x + z * z), two_s * (y * z + x * r)};
    else n = {two_s * (x * z + y * r), two_s * (y * z - x * r), 1.f - two_s * (x * x + y * y)};
    const float3 tc = {campos.x - p.x, campos.y - p.y, campos.z - p.z};
    if (n.x * tc.x + n.y * tc.y + n.z * tc.z < 0.0f) n = {-n.x, -n.y, -n.z};
    const float3 ln = {n.x * V[0] + n.y * V[4] + n.z * V[8], n.x * V[1] + n.y * V[5] + n.z * V[9],
                       n.x * V[2] + n.y * V[6] + n.z * V[10]};
    const float3 pc = {p.x * V[0] + p.y * V[4] + p.z * V[8] + V[12], p.x * V[1] + p.y * V[5] + p.z * V[9] + V[13],
                       p.x * V[2] + p.y * V[6] + p.z * V[10] + V[14]};
    o5[0] = ln.x; o5[1] = ln.y; o5[2] = ln.z; o5[3] = 1.0f;
    o5[4] = fabsf(ln.x * pc.x + ln.y * pc.y + ln.z * pc.z);
}

// Backward of plane_fwd: cotangent g[5] -> ADDED to dp (mean, through the plane distance) and dq (raw quaternion,
// through the chosen rotation column and the normalisation).  The choice of the column, the flip towards the
// camera and the sign of the distance are piecewise constant; scales get no gradient.
__device__ __forceinline__ void plane_bwd(const float3 p, const float3 sc, const float4 qraw, const float* V,
                                          const float3 campos, const float* g, float3& dp, float4& dq)
{
    const float qn = fmaxf(sqrtf(qraw.x * qraw.x + qraw.y * qraw.y + qraw.z * qraw.z + qraw.w * qraw.w), 1e-12f);
    const float r = qraw.x / qn, x = qraw.y / qn, y = qraw.z / qn, z = qraw.w / qn;
    int idx = 0;
    float smin = sc.x;
    if (sc.y < smin) { smin = sc.y; idx = 1; }
    if (sc.z < smin) { smin = sc.z; idx = 2; }
    // on the unit sphere the rotation column is a quadratic form with factor 2
    float3 n;
    if (idx == 0) n = {1.f - 2.f * (y * y + z * z), 2.f * (x * y + z * r), 2.f * (x * z - y * r)};
    else if (idx == 1) n = {2.f * (x * y - z * r), 1.f - 2.f * (x * x + z * z), 2.f * (y * z + x * r)};
    else n = {2.f * (x * z + y * r), 2.f * (y * z - x * r), 1.f - 2.f * (x * x + y * y)};
    const float3 tc = {campos.x - p.x, campos.y - p.y, campos.z - p.z};
    const float flip = (n.x * tc.x + n.y * tc.y + n.z * tc.z < 0.0f) ? -1.f : 1.f;
    n = {flip * n.x, flip * n.y, flip * n.z};
    const float3 ln = {n.x * V[0] + n.y * V[4] + n.z * V[8], n.x * V[1] + n.y * V[5] + n.z * V[9],
                       n.x * V[2] + n.y * V[6] + n.z * V[10]};
    const float3 pc = {p.x * V[0] + p.y * V[4] + p.z * V[8] + V[12], p.x * V[1] + p.y * V[5] + p.z * V[9] + V[13],
                       p.x * V[2] + p.y * V[6] + p.z * V[10] + V[14]};
    const float dot = ln.x * pc.x + ln.y * pc.y + ln.z * pc.z;
    const float gs = dot > 0.f ? g[4] : (dot < 0.f ? -g[4] : 0.f);          // d|t|/dt, 0 at t = 0 as torch.abs
    const float3 dln = {g[0] + gs * pc.x, g[1] + gs * pc.y, g[2] + gs * pc.z};
    const float3 dpc = {gs * ln.x, gs * ln.y, gs * ln.z};
    dp.x += dpc.x * V[0] + dpc.y * V[1] + dpc.z * V[2];
    dp.y += dpc.x * V[4] + dpc.y * V[5] + dpc.z * V[6];
    dp.z += dpc.x * V[8] + dpc.y * V[9] + dpc.z * V[10];
    const float3 dc = {flip * (dln.x * V[0] + dln.y * V[1] + dln.z * V[2]),
                       flip * (dln.x * V[4] + dln.y * V[5] + dln.z * V[6]),
                       flip * (dln.x * V[8] + dln.y * V[9] + dln.z * V[10])};      // cotangent of the column
    float gr, gx, gy, gz;
    if (idx == 0) {
        gr = 2.f * (z * dc.y - y * dc.z);
        gx = 2.f * (y * dc.y + z * dc.z);
        gy = -4.f * y * dc.x + 2.f * (x * dc.y - r * dc.z);
        gz = -4.f * z * dc.x + 2.f * (r * dc.y + x * dc.z);
    } else if (idx == 1) {
        gr = 2.f * (x * dc.z - z * dc.x);
        gx = 2.f * y * dc.x - 4.f * x * dc.y + 2.f * r * dc.z;
        gy = 2.f * (x * dc.x + z * dc.z);
        gz = -2.f * r * dc.x - 4.f * z * dc.y + 2.f * y * dc.z;
    } else {
        gr = 2.f * (y * dc.x - x * dc.y);
        gx = 2.f * z * dc.x - 2.f * r * dc.y - 4.f * x * dc.z;
        gy = 2.f * r * dc.x + 2.f * z * dc.y - 4.f * y * dc.z;
        gz = 2.f * (x * dc.x + y * dc.y);
    }
    // through q / |q|: remove the radial part, divide by the norm
    const float radial = r * gr + x * gx + y * gy + z * gz;
    dq.x += (gr - r * radial) / qn;
    dq.y += (gx - x * radial) / qn;
    dq.z += (gy - y * radial) / qn;
    dq.w += (gz - z * radial) / qn;
}

// radii optional: rows with radius <= 0 (never rasterized) get zeros.
__global__ void __launch_bounds__(256)
all_map_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ scales,
               const float4* __restrict__ rotations, const int* __restrict__ radii,
               const float* __restrict__ viewmatrix, const float* __restrict__ campos, float* __restrict__ out)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P) return;
    float o5[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    if (!radii || radii[i] > 0) {
        const float3 p = {means3D[3 * i], means3D[3 * i + 1], means3D[3 * i + 2]};
        const float3 sc = {scales[3 * i], scales[3 * i + 1], scales[3 * i + 2]};
        plane_fwd(p, sc, rotations[i], viewmatrix, make_float3(campos[0], campos[1], campos[2]), o5);
    }
#pragma unroll
    for (int k = 0; k < 5; k++) out[5 * (size_t)i + k] = o5[k];
}

// dL_dmeans3D / dL_drotations are WRITTEN (rows with radius <= 0 get zeros).
__global__ void __launch_bounds__(256)
all_map_bwd_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ scales,
                   const float4* __restrict__ rotations, const int* __restrict__ radii,
                   const float* __restrict__ viewmatrix, const float* __restrict__ campos,
                   const float* __restrict__ dL_dall_map, float* __restrict__ dL_dmeans3D,
                   float4* __restrict__ dL_drotations)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P) return;
    float3 dp = {0.f, 0.f, 0.f};
    float4 dq = {0.f, 0.f, 0.f, 0.f};
    if (!radii || radii[i] > 0) {
        const float3 p = {means3D[3 * i], means3D[3 * i + 1], means3D[3 * i + 2]};
        const float3 sc = {scales[3 * i], scales[3 * i + 1], scales[3 * i + 2]};
        float g[5];
#pragma unroll
        for (int k = 0; k < 5; k++) g[k] = dL_dall_map[5 * (size_t)i + k];
        plane_bwd(p, sc, rotations[i], viewmatrix, make_float3(campos[0], campos[1], campos[2]), g, dp, dq);
    }
    dL_dmeans3D[3 * (size_t)i] = dp.x;
    dL_dmeans3D[3 * (size_t)i + 1] = dp.y;
    dL_dmeans3D[3 * (size_t)i + 2] = dp.z;
    dL_drotations[i] = dq;
}

// Backward of one camera's projection for one Gaussian: conic cotangent -> 2-D covariance -> (accumulated into)
// dL/dcov3D[6] and dL/dmean, plus the 2-D mean's cotangent through the perspective projection.
__device__ __forceinline__ void bwd_project_one(const float3 mean, const float* cov3D, const float* view_matrix,
                                                const float* proj, const float h_x, const float h_y,
                                                const float tan_fovx, const float tan_fovy, const float4 dco,
                                                const float2 dm2, float3& g_mean, float* dL_dcov)
{
    // ---- conic -> cov2D -> cov3D and mean (EWA part)
    float3 dL_dconic = {dco.x, dco.y, dco.z};
    float3 tt = transform_point_4x3(mean, view_matrix);
    const float limx = 1.3f * tan_fovx;
    const float limy = 1.3f * tan_fovy;
    const float txtz = tt.x / tt.z;
    const float tytz = tt.y / tt.z;
    tt.x = min(limx, max(-limx, txtz)) * tt.z;
    tt.y = min(limy, max(-limy, tytz)) * tt.z;
    const float x_grad_mul = txtz < -limx || txtz > limx ? 0 : 1;
    const float y_grad_mul = tytz < -limy || tytz > limy ? 0 : 1;

    Mat3 J;
    J.m[0][0] = h_x / tt.z; J.m[0][1] = 0.0f; J.m[0][2] = -(h_x * tt.x) / (tt.z * tt.z);
    J.m[1][0] = 0.0f; J.m[1][1] = h_y / tt.z; J.m[1][2] = -(h_y * tt.y) / (tt.z * tt.z);
    J.m[2][0] = 0; J.m[2][1] = 0; J.m[2][2] = 0;
    Mat3 Wm;
    Wm.m[0][0] = view_matrix[0]; Wm.m[0][1] = view_matrix[4]; Wm.m[0][2] = view_matrix[8];
    Wm.m[1][0] = view_matrix[1]; Wm.m[1][1] = view_matrix[5]; Wm.m[1][2] = view_matrix[9];
    Wm.m[2][0] = view_matrix[2]; Wm.m[2][1] = view_matrix[6]; Wm.m[2][2] = view_matrix[10];
    Mat3 Vrk;
    Vrk.m[0][0] = cov3D[0]; Vrk.m[0][1] = cov3D[1]; Vrk.m[0][2] = cov3D[2];
    Vrk.m[1][0] = cov3D[1]; Vrk.m[1][1] = cov3D[3]; Vrk.m[1][2] = cov3D[4];
    Vrk.m[2][0] = cov3D[2]; Vrk.m[2][1] = cov3D[4]; Vrk.m[2][2] = cov3D[5];
    Mat3 T = mul(Wm, J);
    Mat3 cov2D = mul(mul(transpose(T), transpose(Vrk)), T);

    float a = cov2D.m[0][0] += 0.3f;
    float b = cov2D.m[0][1];
    float c = cov2D.m[1][1] += 0.3f;

    float denom = a * c - b * b;
    float dL_da = 0, dL_db = 0, dL_dc = 0;
    float denom2inv = 1.0f / ((denom * denom) + 0.0000001f);
    float dcv[6];
    if (denom2inv != 0) {
        dL_da = denom2inv * (-c * c * dL_dconic.x + 2 * b * c * dL_dconic.y + (denom - a * c) * dL_dconic.z);
        dL_dc = denom2inv * (-a * a * dL_dconic.z + 2 * a * b * dL_dconic.y + (denom - a * c) * dL_dconic.x);
        dL_db = denom2inv * 2 * (b * c * dL_dconic.x - (denom + 2 * b * b) * dL_dconic.y + a * b * dL_dconic.z);

        dcv[0] = (T.m[0][0] * T.m[0][0] * dL_da + T.m[0][0] * T.m[1][0] * dL_db + T.m[1][0] * T.m[1][0] * dL_dc);
        dcv[3] = (T.m[0][1] * T.m[0][1] * dL_da + T.m[0][1] * T.m[1][1] * dL_db + T.m[1][1] * T.m[1][1] * dL_dc);
        dcv[5] = (T.m[0][2] * T.m[0][2] * dL_da + T.m[0][2] * T.m[1][2] * dL_db + T.m[1][2] * T.m[1][2] * dL_dc);
        dcv[1] = 2 * T.m[0][0] * T.m[0][1] * dL_da + (T.m[0][0] * T.m[1][1] + T.m[0][1] * T.m[1][0]) * dL_db + 2 * T.m[1][0] * T.m[1][1] * dL_dc;
        dcv[2] = 2 * T.m[0][0] * T.m[0][2] * dL_da + (T.m[0][0] * T.m[1][2] + T.m[0][2] * T.m[1][0]) * dL_db + 2 * T.m[1][0] * T.m[1][2] * dL_dc;
        dcv[4] = 2 * T.m[0][2] * T.m[0][1] * dL_da + (T.m[0][1] * T.m[1][2] + T.m[0][2] * T.m[1][1]) * dL_db + 2 * T.m[1][1] * T.m[1][2] * dL_dc;
    } else {
#pragma unroll
        for (int i = 0; i < 6; i++) dcv[i] = 0;
    }

    float dL_dT00 = 2 * (T.m[0][0] * Vrk.m[0][0] + T.m[0][1] * Vrk.m[0][1] + T.m[0][2] * Vrk.m[0][2]) * dL_da +
                    (T.m[1][0] * Vrk.m[0][0] + T.m[1][1] * Vrk.m[0][1] + T.m[1][2] * Vrk.m[0][2]) * dL_db;
    float dL_dT01 = 2 * (T.m[0][0] * Vrk.m[1][0] + T.m[0][1] * Vrk.m[1][1] + T.m[0][2] * Vrk.m[1][2]) * dL_da +
                    (T.m[1][0] * Vrk.m[1][0] + T.m[1][1] * Vrk.m[1][1] + T.m[1][2] * Vrk.m[1][2]) * dL_db;
    float dL_dT02 = 2 * (T.m[0][0] * Vrk.m[2][0] + T.m[0][1] * Vrk.m[2][1] + T.m[0][2] * Vrk.m[2][2]) * dL_da +
                    (T.m[1][0] * Vrk.m[2][0] + T.m[1][1] * Vrk.m[2][1] + T.m[1][2] * Vrk.m[2][2]) * dL_db;
    float dL_dT10 = 2 * (T.m[1][0] * Vrk.m[0][0] + T.m[1][1] * Vrk.m[0][1] + T.m[1][2] * Vrk.m[0][2]) * dL_dc +
                    (T.m[0][0] * Vrk.m[0][0] + T.m[0][1] * Vrk.m[0][1] + T.m[0][2] * Vrk.m[0][2]) * dL_db;
    float dL_dT11 = 2 * (T.m[1][0] * Vrk.m[1][0] + T.m[1][1] * Vrk.m[1][1] + T.m[1][2] * Vrk.m[1][2]) * dL_dc +
                    (T.m[0][0] * Vrk.m[1][0] + T.m[0][1] * Vrk.m[1][1] + T.m[0][2] * Vrk.m[1][2]) * dL_db;
    float dL_dT12 = 2 * (T.m[1][0] * Vrk.m[2][0] + T.m[1][1] * Vrk.m[2][1] + T.m[1][2] * Vrk.m[2][2]) * dL_dc +
                    (T.m[0][0] * Vrk.m[2][0] + T.m[0][1] * Vrk.m[2][1] + T.m[0][2] * Vrk.m[2][2]) * dL_db;

    float dL_dJ00 = Wm.m[0][0] * dL_dT00 + Wm.m[0][1] * dL_dT01 + Wm.m[0][2] * dL_dT02;
    float dL_dJ02 = Wm.m[2][0] * dL_dT00 + Wm.m[2][1] * dL_dT01 + Wm.m[2][2] * dL_dT02;
    float dL_dJ11 = Wm.m[1][0] * dL_dT10 + Wm.m[1][1] * dL_dT11 + Wm.m[1][2] * dL_dT12;
    float dL_dJ12 = Wm.m[2][0] * dL_dT10 + Wm.m[2][1] * dL_dT11 + Wm.m[2][2] * dL_dT12;

    float tz = 1.f / tt.z;
    float tz2 = tz * tz;
    float tz3 = tz2 * tz;

    float dL_dtx = x_grad_mul * -h_x * tz2 * dL_dJ02;
    float dL_dty = y_grad_mul * -h_y * tz2 * dL_dJ12;
    float dL_dtz = -h_x * tz2 * dL_dJ00 - h_y * tz2 * dL_dJ11 + (2 * h_x * tt.x) * tz3 * dL_dJ02 + (2 * h_y * tt.y) * tz3 * dL_dJ12;

    float3 dL_dmean = transform_vec_4x3_transpose({dL_dtx, dL_dty, dL_dtz}, view_matrix);

    // ---- projection of the 2-D mean
    float4 m_hom = transform_point_4x4(mean, proj);
    float m_w = 1.0f / (m_hom.w + 0.0000001f);
    float mul1 = (proj[0] * mean.x + proj[4] * mean.y + proj[8] * mean.z + proj[12]) * m_w * m_w;
    float mul2 = (proj[1] * mean.x + proj[5] * mean.y + proj[9] * mean.z + proj[13]) * m_w * m_w;
    float3 dL_dmean_b;
    dL_dmean_b.x = (proj[0] * m_w - proj[3] * mul1) * dm2.x + (proj[1] * m_w - proj[3] * mul2) * dm2.y;
    dL_dmean_b.y = (proj[4] * m_w - proj[7] * mul1) * dm2.x + (proj[5] * m_w - proj[7] * mul2) * dm2.y;
    dL_dmean_b.z = (proj[8] * m_w - proj[11] * mul1) * dm2.x + (proj[9] * m_w - proj[11] * mul2) * dm2.y;
    g_mean.x += dL_dmean.x + dL_dmean_b.x;
        g_mean.y += dL_dmean.y + dL_dmean_b.y;
        g_mean.z += dL_dmean.z + dL_dmean_b.z;
#pragma unroll
        for (int i = 0; i < 6; i++) dL_dcov[i] += dcv[i];
}

// Backward of scale / (unnormalised) quaternion -> 3-D covariance; dL_dcov is the cotangent of its six entries.
__device__ __forceinline__ void bwd_cov3d(const float3 sc, const float scale_modifier, const float4 rot,
                                          const float* dL_dcov, float3& g_scale, float4& g_rot)
{
    // ---- cov3D -> scale, quaternion (quaternion treated as given, not normalised)
    float r = rot.x, x = rot.y, y = rot.z, z = rot.w;
    Mat3 R;
    R.m[0][0] = 1.f - 2.f * (y * y + z * z); R.m[0][1] = 2.f * (x * y - r * z); R.m[0][2] = 2.f * (x * z + r * y);
    R.m[1][0] = 2.f * (x * y + r * z); R.m[1][1] = 1.f - 2.f * (x * x + z * z); R.m[1][2] = 2.f * (y * z - r * x);
    R.m[2][0] = 2.f * (x * z - r * y); R.m[2][1] = 2.f * (y * z + r * x); R.m[2][2] = 1.f - 2.f * (x * x + y * y);
    Mat3 S;
#pragma unroll
    for (int cc = 0; cc < 3; cc++)
#pragma unroll
        for (int rr = 0; rr < 3; rr++) S.m[cc][rr] = 0.0f;
    float3 s = {scale_modifier * sc.x, scale_modifier * sc.y, scale_modifier * sc.z};
    S.m[0][0] = s.x; S.m[1][1] = s.y; S.m[2][2] = s.z;
    Mat3 M = mul(S, R);
    Mat3 dL_dSigma;
    dL_dSigma.m[0][0] = dL_dcov[0]; dL_dSigma.m[0][1] = 0.5f * dL_dcov[1]; dL_dSigma.m[0][2] = 0.5f * dL_dcov[2];
    dL_dSigma.m[1][0] = 0.5f * dL_dcov[1]; dL_dSigma.m[1][1] = dL_dcov[3]; dL_dSigma.m[1][2] = 0.5f * dL_dcov[4];
    dL_dSigma.m[2][0] = 0.5f * dL_dcov[2]; dL_dSigma.m[2][1] = 0.5f * dL_dcov[4]; dL_dSigma.m[2][2] = dL_dcov[5];
    Mat3 M2;
#pragma unroll
    for (int cc = 0; cc < 3; cc++)
#pragma unroll
        for (int rr = 0; rr < 3; rr++) M2.m[cc][rr] = 2.0f * M.m[cc][rr];
    Mat3 dL_dM = mul(M2, dL_dSigma);
    Mat3 Rt = transpose(R);
    Mat3 dL_dMt = transpose(dL_dM);

    g_scale.x = Rt.m[0][0] * dL_dMt.m[0][0] + Rt.m[0][1] * dL_dMt.m[0][1] + Rt.m[0][2] * dL_dMt.m[0][2];
    g_scale.y = Rt.m[1][0] * dL_dMt.m[1][0] + Rt.m[1][1] * dL_dMt.m[1][1] + Rt.m[1][2] * dL_dMt.m[1][2];
    g_scale.z = Rt.m[2][0] * dL_dMt.m[2][0] + Rt.m[2][1] * dL_dMt.m[2][1] + Rt.m[2][2] * dL_dMt.m[2][2];

#pragma unroll
    for (int rr = 0; rr < 3; rr++) {
        dL_dMt.m[0][rr] *= s.x;
        dL_dMt.m[1][rr] *= s.y;
        dL_dMt.m[2][rr] *= s.z;
    }
    g_rot.x = 2 * z * (dL_dMt.m[0][1] - dL_dMt.m[1][0]) + 2 * y * (dL_dMt.m[2][0] - dL_dMt.m[0][2]) + 2 * x * (dL_dMt.m[1][2] - dL_dMt.m[2][1]);
    g_rot.y = 2 * y * (dL_dMt.m[1][0] + dL_dMt.m[0][1]) + 2 * z * (dL_dMt.m[2][0] + dL_dMt.m[0][2]) + 2 * r * (dL_dMt.m[1][2] - dL_dMt.m[2][1]) - 4 * x * (dL_dMt.m[2][2] + dL_dMt.m[1][1]);
    g_rot.z = 2 * x * (dL_dMt.m[1][0] + dL_dMt.m[0][1]) + 2 * r * (dL_dMt.m[2][0] - dL_dMt.m[0][2]) + 2 * z * (dL_dMt.m[1][2] + dL_dMt.m[2][1]) - 4 * y * (dL_dMt.m[2][2] + dL_dMt.m[0][0]);
    g_rot.w = 2 * r * (dL_dMt.m[0][1] - dL_dMt.m[1][0]) + 2 * x * (dL_dMt.m[2][0] + dL_dMt.m[0][2]) + 2 * y * (dL_dMt.m[1][2] + dL_dMt.m[2][1]) - 4 * z * (dL_dMt.m[1][1] + dL_dMt.m[0][0]);
}

// Fused backward of the per-Gaussian stage: d(conic) -> d(cov2D) -> d(cov3D), d(mean) through the EWA
// Jacobian and through the projection of the 2-D mean, then d(cov3D) -> d(scale), d(quaternion).
// The 3-D covariance is recomputed from scale/rotation (same function as the forward, so same bits)
// instead of being read back, and the intermediate dL/dcov3D never leaves registers.
__global__ void __launch_bounds__(CGX_BLOCK_SIZE)
preprocess_bwd_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ scales,
                      const float scale_modifier, const float* __restrict__ rotations,
                      const int* __restrict__ radii, const float* __restrict__ viewmatrix_g,
                      const float* __restrict__ projmatrix_g, const float h_x, float h_y, const float tan_fovx,
                      float tan_fovy, const float2* __restrict__ dL_dmean2D,
                      const float4* __restrict__ dL_dconic_opacity, float* __restrict__ dL_dmeans,
                      float* __restrict__ dL_dscales, float4* __restrict__ dL_drots,
                      float* __restrict__ dL_dopacity, int vec_mask)
{
    __shared__ __align__(16) float s_mean[CGX_BLOCK_SIZE * 3];   // reused for dL_dmeans
    __shared__ __align__(16) float s_scale[CGX_BLOCK_SIZE * 3];  // reused for dL_dscales
    __shared__ __align__(16) float s_rot[CGX_BLOCK_SIZE * 4];
    __shared__ float view_matrix[16];
    __shared__ float proj[16];

    const int base = blockIdx.x * CGX_BLOCK_SIZE;
    const int count = min(CGX_BLOCK_SIZE, P - base);
    if (threadIdx.x < 16) view_matrix[threadIdx.x] = viewmatrix_g[threadIdx.x];
    else if (threadIdx.x < 32) proj[threadIdx.x - 16] = projmatrix_g[threadIdx.x - 16];
    block_load_rows<3>(means3D + (size_t)base * 3, s_mean, count, vec_mask & 1);
    block_load_rows<3>(scales + (size_t)base * 3, s_scale, count, vec_mask & 2);
    block_load_rows<4>(rotations + (size_t)base * 4, s_rot, count, vec_mask & 4);
    __syncthreads();

    const int t = threadIdx.x;
    const int idx = base + t;
    float3 g_mean = {0.f, 0.f, 0.f}, g_scale = {0.f, 0.f, 0.f};
    float4 g_rot = {0.f, 0.f, 0.f, 0.f};

    if (t < count) {
        const float4 dco = __ldg(dL_dconic_opacity + idx);
        dL_dopacity[idx] = dco.w;
        if (radii[idx] > 0) {
            const float3 mean = {s_mean[3 * t], s_mean[3 * t + 1], s_mean[3 * t + 2]};
            const float3 sc = {s_scale[3 * t], s_scale[3 * t + 1], s_scale[3 * t + 2]};
            const float4 rot = {s_rot[4 * t], s_rot[4 * t + 1], s_rot[4 * t + 2], s_rot[4 * t + 3]};
            float cov3D[6];
            compute_cov3d(sc, scale_modifier, rot, cov3D);

            float dL_dcov[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            bwd_project_one(mean, cov3D, view_matrix, proj, h_x, h_y, tan_fovx, tan_fovy, dco,
                            __ldg(dL_dmean2D + idx), g_mean, dL_dcov);
            bwd_cov3d(sc, scale_modifier, rot, dL_dcov, g_scale, g_rot);
        }
        dL_drots[idx] = g_rot;
    }
    __syncthreads();  // everyone is done reading s_mean / s_scale
    if (t < count) {
        s_mean[3 * t] = g_mean.x; s_mean[3 * t + 1] = g_mean.y; s_mean[3 * t + 2] = g_mean.z;
        s_scale[3 * t] = g_scale.x; s_scale[3 * t + 1] = g_scale.y; s_scale[3 * t + 2] = g_scale.z;
    }
    __syncthreads();
    block_store_rows<3>(dL_dmeans + (size_t)base * 3, s_mean, count, vec_mask & 8);
    block_store_rows<3>(dL_dscales + (size_t)base * 3, s_scale, count, vec_mask & 16);
}

// ------------------------------------------------------------------------------------------------ batched over cameras
// The caller's per-camera loop around preprocess (gaussian_renderer/__init__.py:966-1023) as one launch: every
// Gaussian's parameters are read ONCE and projected into all B cameras of the batch; the backward reads them once
// and writes the gradients summed over the cameras once (instead of B partial results added up by autograd).
constexpr int MAX_CAMS = 16;

struct CamBatch {
    int B;
    const float* view[MAX_CAMS];   // device pointers to the 4x4 matrices
    const float* proj[MAX_CAMS];
    float tan_fovx[MAX_CAMS], tan_fovy[MAX_CAMS], focal_x[MAX_CAMS], focal_y[MAX_CAMS];
    int W[MAX_CAMS], H[MAX_CAMS];
};
struct CamOutputs {
    float2* means2D[MAX_CAMS];
    float* depths[MAX_CAMS];
    int* radii[MAX_CAMS];
    float4* conic_opacity[MAX_CAMS];
};
struct CamCotangents {
    const int* radii[MAX_CAMS];
    const float2* dL_dmeans2D[MAX_CAMS];
    const float4* dL_dconic_opacity[MAX_CAMS];
};
// Optional plane descriptors per camera: forward output (P,5) / backward cotangent (P,5); null = not wanted.
struct CamPlanes {
    const float* campos[MAX_CAMS];
    float* all_map[MAX_CAMS];
    const float* dL_dall_map[MAX_CAMS];
};

__global__ void __launch_bounds__(CGX_BLOCK_SIZE)
preprocess_fwd_batched_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ scales,
                              const float scale_modifier, const float* __restrict__ rotations,
                              const float* __restrict__ opacities, CamBatch cams, CamOutputs outs, CamPlanes planes,
                              int vec_mask)
{
    __shared__ __align__(16) float s_mean[CGX_BLOCK_SIZE * 3];
    __shared__ __align__(16) float s_scale[CGX_BLOCK_SIZE * 3];
    __shared__ __align__(16) float s_rot[CGX_BLOCK_SIZE * 4];
    __shared__ float s_view[MAX_CAMS][16];
    __shared__ float s_proj[MAX_CAMS][16];

    const int base = blockIdx.x * CGX_BLOCK_SIZE;
    const int count = min(CGX_BLOCK_SIZE, P - base);
    for (int i = threadIdx.x; i < cams.B * 32; i += blockDim.x) {
        const int b = i >> 5, e = i & 31;
        if (e < 16) s_view[b][e] = cams.view[b][e];
        else s_proj[b][e - 16] = cams.proj[b][e - 16];
    }
    block_load_rows<3>(means3D + (size_t)base * 3, s_mean, count, vec_mask & 1);
    block_load_rows<3>(scales + (size_t)base * 3, s_scale, count, vec_mask & 2);
    block_load_rows<4>(rotations + (size_t)base * 4, s_rot, count, vec_mask & 4);
    __syncthreads();

    const int t = threadIdx.x;
    if (t >= count) return;
    const int idx = base + t;
    const float3 p_orig = {s_mean[3 * t], s_mean[3 * t + 1], s_mean[3 * t + 2]};
    const float3 sc = {s_scale[3 * t], s_scale[3 * t + 1], s_scale[3 * t + 2]};
    const float4 q = {s_rot[4 * t], s_rot[4 * t + 1], s_rot[4 * t + 2], s_rot[4 * t + 3]};
    const float opacity = __ldg(opacities + idx);
    float cov3D[6];
    compute_cov3d(sc, scale_modifier, q, cov3D);   // camera independent

#pragma unroll 1
    for (int b = 0; b < cams.B; b++) {
        const float* viewmatrix = s_view[b];
        const float* projmatrix = s_proj[b];
        const int W = cams.W[b], H = cams.H[b];
        int out_radius = 0;
        float2 out_xy = {0.f, 0.f};
        float out_depth = 0.f;
        float4 out_co = {0.f, 0.f, 0.f, 0.f};
        do {
            float4 p_hom = transform_point_4x4(p_orig, projmatrix);
            float p_w = 1.0f / (p_hom.w + 0.0000001f);
            float3 p_proj = {p_hom.x * p_w, p_hom.y * p_w, p_hom.z * p_w};
            float3 p_view = transform_point_4x3(p_orig, viewmatrix);
            if (p_view.z <= 0.0f) break;
            float3 cov = compute_cov2d(p_orig, cams.focal_x[b], cams.focal_y[b], cams.tan_fovx[b], cams.tan_fovy[b],
                                       cov3D, viewmatrix);
            float det = (cov.x * cov.z - cov.y * cov.y);
            if (det == 0.0f) break;
            float det_inv = 1.f / det;
            float3 conic = {cov.z * det_inv, -cov.y * det_inv, cov.x * det_inv};
            float mid = 0.5f * (cov.x + cov.z);
            float lambda1 = mid + sqrt(max(0.1f, mid * mid - det));
            float lambda2 = mid - sqrt(max(0.1f, mid * mid - det));
            float my_radius = ceil(3.f * sqrt(max(lambda1, lambda2)));
            float2 point_image = {ndc2pix(p_proj.x, W), ndc2pix(p_proj.y, H)};
            uint2 rect_min, rect_max;
            get_rect(point_image, my_radius, rect_min, rect_max, (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X,
                     (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y);
            if ((rect_max.x - rect_min.x) * (rect_max.y - rect_min.y) == 0) break;
            out_depth = p_view.z;
            out_radius = my_radius;
            out_xy = point_image;
            out_co = {conic.x, conic.y, conic.z, opacity};
        } while (0);
        outs.radii[b][idx] = out_radius;
        outs.means2D[b][idx] = out_xy;
        outs.depths[b][idx] = out_depth;
        outs.conic_opacity[b][idx] = out_co;
        if (planes.all_map[b]) {
            float o5[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
            if (out_radius > 0) {
                const float* cp = planes.campos[b];
                plane_fwd(p_orig, sc, q, viewmatrix, make_float3(__ldg(cp), __ldg(cp + 1), __ldg(cp + 2)), o5);
            }
            float* o = planes.all_map[b] + 5 * (size_t)idx;
#pragma unroll
            for (int k = 0; k < 5; k++) o[k] = o5[k];
        }
    }
}

#ifndef CGX_PRE_BWD_COMPACT
#define CGX_PRE_BWD_COMPACT 1     // 1: the CTA-compacted kernel below serves cgx_preprocess_bwd_batched*; 0: the walk per Gaussian
#endif
#ifndef CGX_PRE_BWD_MIN_CTAS
#define CGX_PRE_BWD_MIN_CTAS 3
#endif
// 3 CTAs per SM: the kernel is latency-bound (dependent divisions and square roots per camera), so the third CTA's
// warps matter more than the registers it costs.
__global__ void __launch_bounds__(CGX_BLOCK_SIZE, CGX_PRE_BWD_MIN_CTAS)
preprocess_bwd_batched_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ scales,
                              const float scale_modifier, const float* __restrict__ rotations, CamBatch cams,
                              CamCotangents cot, CamPlanes planes, float* __restrict__ dL_dmeans,
                              float* __restrict__ dL_dscales, float4* __restrict__ dL_drots,
                              float* __restrict__ dL_dopacity, int vec_mask)
{
    __shared__ __align__(16) float s_mean[CGX_BLOCK_SIZE * 3];   // reused for dL_dmeans
    __shared__ __align__(16) float s_scale[CGX_BLOCK_SIZE * 3];  // reused for dL_dscales
    __shared__ __align__(16) float s_rot[CGX_BLOCK_SIZE * 4];
    __shared__ float s_view[MAX_CAMS][16];
    __shared__ float s_proj[MAX_CAMS][16];

    const int base = blockIdx.x * CGX_BLOCK_SIZE;
    const int count = min(CGX_BLOCK_SIZE, P - base);
    for (int i = threadIdx.x; i < cams.B * 32; i += blockDim.x) {
        const int b = i >> 5, e = i & 31;
        if (e < 16) s_view[b][e] = cams.view[b][e];
        else s_proj[b][e - 16] = cams.proj[b][e - 16];
    }
    block_load_rows<3>(means3D + (size_t)base * 3, s_mean, count, vec_mask & 1);
    block_load_rows<3>(scales + (size_t)base * 3, s_scale, count, vec_mask & 2);
    block_load_rows<4>(rotations + (size_t)base * 4, s_rot, count, vec_mask & 4);
    __syncthreads();

    const int t = threadIdx.x;
    const int idx = base + t;
    float3 g_mean = {0.f, 0.f, 0.f}, g_scale = {0.f, 0.f, 0.f};
    float4 g_rot = {0.f, 0.f, 0.f, 0.f};
    if (t < count) {
        const float3 mean = {s_mean[3 * t], s_mean[3 * t + 1], s_mean[3 * t + 2]};
        const float3 sc = {s_scale[3 * t], s_scale[3 * t + 1], s_scale[3 * t + 2]};
        const float4 rot = {s_rot[4 * t], s_rot[4 * t + 1], s_rot[4 * t + 2], s_rot[4 * t + 3]};
        float cov3D[6];
        compute_cov3d(sc, scale_modifier, rot, cov3D);
        float dL_dcov[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float g_op = 0.f;
        bool any = false;
        float4 g_rot_plane = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int b = 0; b < cams.B; b++) {
            const float4 dco = __ldg(cot.dL_dconic_opacity[b] + idx);
            g_op += dco.w;
            if (cot.radii[b][idx] > 0) {
                any = true;
                bwd_project_one(mean, cov3D, s_view[b], s_proj[b], cams.focal_x[b], cams.focal_y[b], cams.tan_fovx[b],
                                cams.tan_fovy[b], dco, __ldg(cot.dL_dmeans2D[b] + idx), g_mean, dL_dcov);
                if (planes.dL_dall_map[b]) {
                    const float* gp = planes.dL_dall_map[b] + 5 * (size_t)idx;
                    const float g5[5] = {__ldg(gp), __ldg(gp + 1), __ldg(gp + 2), __ldg(gp + 3), __ldg(gp + 4)};
                    const float* cp = planes.campos[b];
                    plane_bwd(mean, sc, rot, s_view[b], make_float3(__ldg(cp), __ldg(cp + 1), __ldg(cp + 2)), g5,
                              g_mean, g_rot_plane);
                }
            }
        }
        if (any) bwd_cov3d(sc, scale_modifier, rot, dL_dcov, g_scale, g_rot);   // linear in dL_dcov: once for all cameras
        g_rot = {g_rot.x + g_rot_plane.x, g_rot.y + g_rot_plane.y, g_rot.z + g_rot_plane.z, g_rot.w + g_rot_plane.w};
        dL_dopacity[idx] = g_op;
        dL_drots[idx] = g_rot;
    }
    __syncthreads();
    if (t < count) {
        s_mean[3 * t] = g_mean.x; s_mean[3 * t + 1] = g_mean.y; s_mean[3 * t + 2] = g_mean.z;
        s_scale[3 * t] = g_scale.x; s_scale[3 * t + 1] = g_scale.y; s_scale[3 * t + 2] = g_scale.z;
    }
    __syncthreads();
    block_store_rows<3>(dL_dmeans + (size_t)base * 3, s_mean, count, vec_mask & 8);
    block_store_rows<3>(dL_dscales + (size_t)base * 3, s_scale, count, vec_mask & 16);
}

// The same backward with the work compacted inside the CTA.  In the kernel above a thread owns a Gaussian and walks
// the cameras; a Gaussian is visible in a minority of them and its neighbours in memory are visible in OTHER ones, so
// most lanes of a warp idle through every camera's arithmetic.  Here the CTA first lists its visible (Gaussian,
// camera) pairs in shared memory, then its threads work through the list (every lane busy) and add each pair's
// partial results to per-Gaussian sums in shared memory; the covariance backward and the stores follow per Gaussian.
constexpr int PRE_ACC = 15;      // floats per Gaussian: dL/dmean 3 | dL/dcov3D 6 | plane dL/drot 4 | dL/dopacity 1, odd pitch
#ifndef CGX_PRE_BWDC_MIN_CTAS
#define CGX_PRE_BWDC_MIN_CTAS 4
#endif
__global__ void __launch_bounds__(CGX_BLOCK_SIZE, CGX_PRE_BWDC_MIN_CTAS)
preprocess_bwd_batched_compact_kernel(int P, const float* __restrict__ means3D, const float* __restrict__ scales,
                                      const float scale_modifier, const float* __restrict__ rotations,
                                      const __grid_constant__ CamBatch cams, const __grid_constant__ CamCotangents cot,
                                      const __grid_constant__ CamPlanes planes, float* __restrict__ dL_dmeans,
                                      float* __restrict__ dL_dscales, float4* __restrict__ dL_drots,
                                      float* __restrict__ dL_dopacity, int vec_mask)
{
    __shared__ __align__(16) float s_mean[CGX_BLOCK_SIZE * 3];   // reused for dL_dmeans
    __shared__ __align__(16) float s_scale[CGX_BLOCK_SIZE * 3];  // reused for dL_dscales
    __shared__ __align__(16) float s_rot[CGX_BLOCK_SIZE * 4];
    __shared__ float s_cov[CGX_BLOCK_SIZE * 6 + 1];
    __shared__ float s_acc[CGX_BLOCK_SIZE * PRE_ACC];
    __shared__ float s_view[MAX_CAMS][16];
    __shared__ float s_proj[MAX_CAMS][16];
    __shared__ uint16_t s_list[CGX_BLOCK_SIZE * MAX_CAMS];       // (camera << 8) | Gaussian of the CTA
    __shared__ int s_count;

    const int base = blockIdx.x * CGX_BLOCK_SIZE;
    const int count = min(CGX_BLOCK_SIZE, P - base);
    const int t = threadIdx.x, lane = t & 31;
    for (int i = t; i < cams.B * 32; i += blockDim.x) {
        const int b = i >> 5, e = i & 31;
        if (e < 16) s_view[b][e] = cams.view[b][e];
        else s_proj[b][e - 16] = cams.proj[b][e - 16];
    }
    for (int i = t; i < CGX_BLOCK_SIZE * PRE_ACC; i += blockDim.x) s_acc[i] = 0.f;
    if (t == 0) s_count = 0;
    block_load_rows<3>(means3D + (size_t)base * 3, s_mean, count, vec_mask & 1);
    block_load_rows<3>(scales + (size_t)base * 3, s_scale, count, vec_mask & 2);
    block_load_rows<4>(rotations + (size_t)base * 4, s_rot, count, vec_mask & 4);
    __syncthreads();

    // ---- list the visible pairs (warp-aggregated append; the order inside the list does not matter)
    const int idx = base + t;
    if (t < count) {
        const float3 sc = {s_scale[3 * t], s_scale[3 * t + 1], s_scale[3 * t + 2]};
        const float4 rot = {s_rot[4 * t], s_rot[4 * t + 1], s_rot[4 * t + 2], s_rot[4 * t + 3]};
        float cov3D[6];
        compute_cov3d(sc, scale_modifier, rot, cov3D);
#pragma unroll
        for (int k = 0; k < 6; k++) s_cov[6 * t + k] = cov3D[k];
    }
    // all radii first, then the opacity cotangents of the cameras this Gaussian is not visible in (the reference's
    // glue returns a plain slice of dL/dconic_opacity, whatever the radius): independent loads, two round trips
    uint32_t vis_mask = 0;
#pragma unroll
    for (int b = 0; b < MAX_CAMS; b++)
        if (b < cams.B && t < count && __ldg(cot.radii[b] + idx) > 0) vis_mask |= 1u << b;
    float g_op_rest = 0.f;
#pragma unroll
    for (int b = 0; b < MAX_CAMS; b++)
        if (b < cams.B && t < count && !((vis_mask >> b) & 1u))
            g_op_rest += __ldg(reinterpret_cast<const float*>(cot.dL_dconic_opacity[b] + idx) + 3);
    for (int b = 0; b < cams.B; b++) {
        const bool vis = (vis_mask >> b) & 1u;
        const uint32_t m = __ballot_sync(0xffffffffu, vis);
        if (m) {
            int at = 0;
            if (lane == 0) at = atomicAdd(&s_count, __popc(m));
            at = __shfl_sync(0xffffffffu, at, 0);
            if (vis) s_list[at + __popc(m & ((1u << lane) - 1u))] = (uint16_t)((b << 8) | t);
        }
    }
    __syncthreads();

    // ---- one pair per thread and turn
    const int n_pairs = s_count;
    for (int p = t; p < n_pairs; p += CGX_BLOCK_SIZE) {
        const int e = s_list[p];
        const int b = e >> 8, g = e & 255;
        const int gi = base + g;
        const float3 mean = {s_mean[3 * g], s_mean[3 * g + 1], s_mean[3 * g + 2]};
        float cov3D[6];
#pragma unroll
        for (int k = 0; k < 6; k++) cov3D[k] = s_cov[6 * g + k];
        const float4 dco = __ldg(cot.dL_dconic_opacity[b] + gi);
        const float2 dm2 = __ldg(cot.dL_dmeans2D[b] + gi);
        float3 g_mean = {0.f, 0.f, 0.f};
        float dL_dcov[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float4 g_rot_plane = {0.f, 0.f, 0.f, 0.f};
        bwd_project_one(mean, cov3D, s_view[b], s_proj[b], cams.focal_x[b], cams.focal_y[b], cams.tan_fovx[b],
                        cams.tan_fovy[b], dco, dm2, g_mean, dL_dcov);
        if (planes.dL_dall_map[b]) {
            const float3 sc = {s_scale[3 * g], s_scale[3 * g + 1], s_scale[3 * g + 2]};
            const float4 rot = {s_rot[4 * g], s_rot[4 * g + 1], s_rot[4 * g + 2], s_rot[4 * g + 3]};
            const float* gp = planes.dL_dall_map[b] + 5 * (size_t)gi;
            const float g5[5] = {__ldg(gp), __ldg(gp + 1), __ldg(gp + 2), __ldg(gp + 3), __ldg(gp + 4)};
            const float* cp = planes.campos[b];
            plane_bwd(mean, sc, rot, s_view[b], make_float3(__ldg(cp), __ldg(cp + 1), __ldg(cp + 2)), g5, g_mean,
                      g_rot_plane);
        }
        float* a = s_acc + g * PRE_ACC;
        atomicAdd(a + 0, g_mean.x); atomicAdd(a + 1, g_mean.y); atomicAdd(a + 2, g_mean.z);
#pragma unroll
        for (int k = 0; k < 6; k++) atomicAdd(a + 3 + k, dL_dcov[k]);
        atomicAdd(a + 9, g_rot_plane.x); atomicAdd(a + 10, g_rot_plane.y);
        atomicAdd(a + 11, g_rot_plane.z); atomicAdd(a + 12, g_rot_plane.w);
        atomicAdd(a + 13, dco.w);
    }
    __syncthreads();

    // ---- per Gaussian: covariance backward (linear in dL/dcov3D: once for all cameras) and the stores
    float3 g_mean = {0.f, 0.f, 0.f}, g_scale = {0.f, 0.f, 0.f};
    if (t < count) {
        const float* a = s_acc + t * PRE_ACC;
        const float g_op = a[13] + g_op_rest;
        float dL_dcov[6];
        bool any = false;
#pragma unroll
        for (int k = 0; k < 6; k++) {
            dL_dcov[k] = a[3 + k];
            any |= dL_dcov[k] != 0.f;
        }
        float4 g_rot = {0.f, 0.f, 0.f, 0.f};
        if (any) {
            const float3 sc = {s_scale[3 * t], s_scale[3 * t + 1], s_scale[3 * t + 2]};
            const float4 rot = {s_rot[4 * t], s_rot[4 * t + 1], s_rot[4 * t + 2], s_rot[4 * t + 3]};
            bwd_cov3d(sc, scale_modifier, rot, dL_dcov, g_scale, g_rot);
        }
        g_mean = {a[0], a[1], a[2]};
        dL_dopacity[idx] = g_op;
        dL_drots[idx] = {g_rot.x + a[9], g_rot.y + a[10], g_rot.z + a[11], g_rot.w + a[12]};
    }
    __syncthreads();
    if (t < count) {
        s_mean[3 * t] = g_mean.x; s_mean[3 * t + 1] = g_mean.y; s_mean[3 * t + 2] = g_mean.z;
        s_scale[3 * t] = g_scale.x; s_scale[3 * t + 1] = g_scale.y; s_scale[3 * t + 2] = g_scale.z;
    }
    __syncthreads();
    block_store_rows<3>(dL_dmeans + (size_t)base * 3, s_mean, count, vec_mask & 8);
    block_store_rows<3>(dL_dscales + (size_t)base * 3, s_scale, count, vec_mask & 16);
}

// ------------------------------------------------------------------------------------------------ row-driven backward
// The owner's backward over the gradient rows that came back from the ranks that rendered its Gaussians (the
// exchange's reverse leg): one thread per returned row instead of one per (Gaussian, camera) pair.  Only pairs that
// were visible somewhere do any work, a Gaussian that went to two ranks for one camera simply has two rows, and no
// dense per-camera cotangent arrays are built.  Per-Gaussian partial results are summed with 16-byte vector atomics
// in a (P,16) table [dL/dmean 3 | dL/dcov3D 6 | dL/drot from the plane descriptors 4 | dL/dopacity 1 | 2 unused]; a second kernel runs the
// covariance backward once per Gaussian (it is linear in dL/dcov3D) and writes the parameter gradients.
constexpr int MAX_ROW_SEGS = 64;
constexpr int ROW_ACC = 16;      // floats per Gaussian in the table: 14 used, rows stay 16-byte aligned for vector atomics
struct RowSegments {
    long long start[MAX_ROW_SEGS];   // first row of the segment in the row table
    int count[MAX_ROW_SEGS];
    int cam[MAX_ROW_SEGS];           // camera the segment's rows belong to
};

template <int NCOLS>   // 14: means2D 2 | rgb 3 | conic_opacity 4 | plane descriptors 5;  9: without the descriptors
__global__ void __launch_bounds__(256, 4)
preprocess_bwd_rows_kernel(const __grid_constant__ RowSegments segs, const float* __restrict__ rows,
                           const int* __restrict__ row_gaussian, const float* __restrict__ means3D,
                           const float* __restrict__ scales, const float scale_modifier,
                           const float4* __restrict__ rotations, const __grid_constant__ CamBatch cams,
                           const __grid_constant__ CamPlanes planes, float* __restrict__ acc)
{
    const int s = blockIdx.y;
    const int n = segs.count[s];
    if ((int)blockIdx.x * 256 >= n) return;                 // uniform over the CTA
    const int b = segs.cam[s];
    __shared__ float s_view[16], s_proj[16];
    if (threadIdx.x < 16) s_view[threadIdx.x] = cams.view[b][threadIdx.x];
    else if (threadIdx.x < 32) s_proj[threadIdx.x - 16] = cams.proj[b][threadIdx.x - 16];
    __syncthreads();
    // the CTA's rows are one contiguous piece of the table: staged with coalesced loads
    __shared__ float s_rows[256 * NCOLS];
    const int n_cta = min(256, n - (int)blockIdx.x * 256);
    const float* src = rows + (segs.start[s] + (long long)blockIdx.x * 256) * NCOLS;
    for (int e = threadIdx.x; e < n_cta * NCOLS; e += 256) s_rows[e] = __ldg(src + e);
    __syncthreads();
    const int r = blockIdx.x * 256 + threadIdx.x;
    if (r >= n) return;
    const long long row = segs.start[s] + r;
    const int i = __ldg(row_gaussian + row);
    const float* g = s_rows + threadIdx.x * NCOLS;
    const float2 dm2 = {g[0], g[1]};
    const float4 dco = {g[5], g[6], g[7], g[8]};
    const float3 mean = {__ldg(means3D + 3 * (size_t)i), __ldg(means3D + 3 * (size_t)i + 1),
                         __ldg(means3D + 3 * (size_t)i + 2)};
    const float3 sc = {__ldg(scales + 3 * (size_t)i), __ldg(scales + 3 * (size_t)i + 1),
                       __ldg(scales + 3 * (size_t)i + 2)};
    const float4 rot = __ldg(rotations + i);
    float cov3D[6];
    compute_cov3d(sc, scale_modifier, rot, cov3D);
    float3 g_mean = {0.f, 0.f, 0.f};
    float dL_dcov[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float4 g_rot_plane = {0.f, 0.f, 0.f, 0.f};
    bwd_project_one(mean, cov3D, s_view, s_proj, cams.focal_x[b], cams.focal_y[b], cams.tan_fovx[b],
                    cams.tan_fovy[b], dco, dm2, g_mean, dL_dcov);
    if (NCOLS == 14 && planes.campos[b]) {
        const float g5[5] = {g[9], g[10], g[11], g[12], g[13]};
        const float* cp = planes.campos[b];
        plane_bwd(mean, sc, rot, s_view, make_float3(__ldg(cp), __ldg(cp + 1), __ldg(cp + 2)), g5, g_mean,
                  g_rot_plane);
    }
    float4* a = reinterpret_cast<float4*>(acc + (size_t)i * ROW_ACC);
    atomicAdd(a + 0, make_float4(g_mean.x, g_mean.y, g_mean.z, dL_dcov[0]));
    atomicAdd(a + 1, make_float4(dL_dcov[1], dL_dcov[2], dL_dcov[3], dL_dcov[4]));
    atomicAdd(a + 2, make_float4(dL_dcov[5], g_rot_plane.x, g_rot_plane.y, g_rot_plane.z));
    atomicAdd(a + 3, make_float4(g_rot_plane.w, dco.w, 0.f, 0.f));
}

__global__ void __launch_bounds__(256)
preprocess_bwd_rows_finish_kernel(int P, const float* __restrict__ scales, const float scale_modifier,
                                  const float4* __restrict__ rotations, const float* __restrict__ acc,
                                  float* __restrict__ dL_dmeans, float* __restrict__ dL_dscales,
                                  float4* __restrict__ dL_drots, float* __restrict__ dL_dopacity)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P) return;
    const float* a = acc + (size_t)i * ROW_ACC;
    float dL_dcov[6];
    bool any = false;
#pragma unroll
    for (int k = 0; k < 6; k++) {
        dL_dcov[k] = a[3 + k];
        any |= dL_dcov[k] != 0.f;
    }
    float3 g_scale = {0.f, 0.f, 0.f};
    float4 g_rot = {0.f, 0.f, 0.f, 0.f};
    if (any) {
        const float3 sc = {scales[3 * (size_t)i], scales[3 * (size_t)i + 1], scales[3 * (size_t)i + 2]};
        bwd_cov3d(sc, scale_modifier, rotations[i], dL_dcov, g_scale, g_rot);
    }
    dL_dmeans[3 * (size_t)i] = a[0]; dL_dmeans[3 * (size_t)i + 1] = a[1]; dL_dmeans[3 * (size_t)i + 2] = a[2];
    dL_dscales[3 * (size_t)i] = g_scale.x; dL_dscales[3 * (size_t)i + 1] = g_scale.y;
    dL_dscales[3 * (size_t)i + 2] = g_scale.z;
    dL_drots[i] = {g_rot.x + a[9], g_rot.y + a[10], g_rot.z + a[11], g_rot.w + a[12]};
    dL_dopacity[i] = a[13];
}

}  // namespace cgx


using namespace cgx;

extern "C" int cgx_mark_visible(int P, const float* means3D, const float* viewmatrix, uint8_t* present, void* stream)
{
    if (P < 0) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means3D || !viewmatrix || !present) return CGX_EINVAL;
    mark_visible_kernel<<<(P + 255) / 256, 256, 0, (cudaStream_t)stream>>>(P, means3D, viewmatrix, present);
    return check_launch();
}

static int preprocess_launch(bool filter, int P, const float* means3D, const float* scales, float scale_modifier,
                             const float* rotations, const float* opacities, const float* viewmatrix,
                             const float* projmatrix, int W, int H, float tanfovx, float tanfovy, float* means2D,
                             float* depths, int32_t* radii, float* cov3D, float* conic_opacity, void* stream,
                             const float* cov3D_precomp = nullptr)
{
    if (P < 0 || W <= 0 || H <= 0) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means3D || !viewmatrix || !projmatrix || !radii) return CGX_EINVAL;
    if (!(filter && cov3D_precomp) && (!scales || !rotations)) return CGX_EINVAL;
    if (!filter && (!opacities || !means2D || !depths || !cov3D || !conic_opacity)) return CGX_EINVAL;
    if (!filter && (((uintptr_t)means2D & 7) || !aligned16(conic_opacity))) return CGX_EINVAL;
    // focal lengths are computed on the host in fp32, as the reference does before launching
    const float focal_y = H / (2.0f * tanfovy);
    const float focal_x = W / (2.0f * tanfovx);
    const int vec_mask = (aligned16(means3D) ? 1 : 0) | (aligned16(scales) ? 2 : 0) | (aligned16(rotations) ? 4 : 0) |
                         ((!filter && aligned16(cov3D)) ? 8 : 0);
    const int grid = (P + CGX_BLOCK_SIZE - 1) / CGX_BLOCK_SIZE;
    cudaStream_t st = (cudaStream_t)stream;
    if (filter)
        preprocess_fwd_kernel<true><<<grid, CGX_BLOCK_SIZE, 0, st>>>(
            P, means3D, scales, scale_modifier, rotations, opacities, viewmatrix, projmatrix, W, H, tanfovx, tanfovy,
            focal_x, focal_y, radii, (float2*)means2D, depths, cov3D, (float4*)conic_opacity, vec_mask, cov3D_precomp);
    else
        preprocess_fwd_kernel<false><<<grid, CGX_BLOCK_SIZE, 0, st>>>(
            P, means3D, scales, scale_modifier, rotations, opacities, viewmatrix, projmatrix, W, H, tanfovx, tanfovy,
            focal_x, focal_y, radii, (float2*)means2D, depths, cov3D, (float4*)conic_opacity, vec_mask, nullptr);
    return check_launch();
}

extern "C" int cgx_preprocess_fwd(int P, const float* means3D, const float* scales, float scale_modifier,
                                  const float* rotations, const float* opacities, const float* viewmatrix,
                                  const float* projmatrix, int W, int H, float tanfovx, float tanfovy,
                                  float* means2D, float* depths, int32_t* radii, float* cov3D, float* conic_opacity,
                                  void* stream)
{
    return preprocess_launch(false, P, means3D, scales, scale_modifier, rotations, opacities, viewmatrix, projmatrix,
                             W, H, tanfovx, tanfovy, means2D, depths, radii, cov3D, conic_opacity, stream);
}

extern "C" int cgx_filter_preprocess(int P, const float* means3D, const float* scales, float scale_modifier,
                                     const float* rotations, const float* viewmatrix, const float* projmatrix,
                                     int W, int H, float tanfovx, float tanfovy, int32_t* radii, void* stream)
{
    return preprocess_launch(true, P, means3D, scales, scale_modifier, rotations, nullptr, viewmatrix, projmatrix, W,
                             H, tanfovx, tanfovy, nullptr, nullptr, radii, nullptr, nullptr, stream);
}

extern "C" int cgx_filter_preprocess_cov3d(int P, const float* means3D, const float* cov3D_precomp,
                                           const float* viewmatrix, const float* projmatrix, int W, int H,
                                           float tanfovx, float tanfovy, int32_t* radii, void* stream)
{
    if (P > 0 && !cov3D_precomp) return CGX_EINVAL;
    return preprocess_launch(true, P, means3D, nullptr, 1.0f, nullptr, nullptr, viewmatrix, projmatrix, W, H, tanfovx,
                             tanfovy, nullptr, nullptr, radii, nullptr, nullptr, stream, cov3D_precomp);
}

extern "C" int cgx_sh_to_rgb(int P, int degree, int M, const float* means3D, const float* campos, const float* sh,
                             float* rgb, uint8_t* clamped, void* stream)
{
    if (P < 0 || degree < 0 || degree > 3 || M < (degree + 1) * (degree + 1) || M > 16) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means3D || !campos || !sh || !rgb || !clamped) return CGX_EINVAL;
    const size_t smem = (size_t)128 * M * 3 * sizeof(float);
    sh_to_rgb_kernel<<<(P + 127) / 128, 128, smem, (cudaStream_t)stream>>>(P, degree, M, means3D, campos, sh, rgb,
                                                                          clamped, aligned16(sh) ? 1 : 0);
    return check_launch();
}

extern "C" int cgx_preprocess_bwd(int P, const float* means3D, const float* scales, float scale_modifier,
                                  const float* rotations, const int32_t* radii, const float* viewmatrix,
                                  const float* projmatrix, int W, int H, float tanfovx, float tanfovy,
                                  const float* dL_dmeans2D, const float* dL_dconic_opacity, float* dL_dmeans3D,
                                  float* dL_dscales, float* dL_drotations, float* dL_dopacity, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means3D || !scales || !rotations || !radii || !viewmatrix || !projmatrix || !dL_dmeans2D ||
        !dL_dconic_opacity || !dL_dmeans3D || !dL_dscales || !dL_drotations || !dL_dopacity)
        return CGX_EINVAL;
    if (((uintptr_t)dL_dmeans2D & 7) || !aligned16(dL_dconic_opacity) || !aligned16(dL_drotations)) return CGX_EINVAL;
    const float focal_y = H / (2.0f * tanfovy);
    const float focal_x = W / (2.0f * tanfovx);
    const int vec_mask = (aligned16(means3D) ? 1 : 0) | (aligned16(scales) ? 2 : 0) | (aligned16(rotations) ? 4 : 0) |
                         (aligned16(dL_dmeans3D) ? 8 : 0) | (aligned16(dL_dscales) ? 16 : 0);
    preprocess_bwd_kernel<<<(P + CGX_BLOCK_SIZE - 1) / CGX_BLOCK_SIZE, CGX_BLOCK_SIZE, 0, (cudaStream_t)stream>>>(
        P, means3D, scales, scale_modifier, rotations, radii, viewmatrix, projmatrix, focal_x, focal_y, tanfovx,
        tanfovy, (const float2*)dL_dmeans2D, (const float4*)dL_dconic_opacity, dL_dmeans3D, dL_dscales,
        (float4*)dL_drotations, dL_dopacity, vec_mask);
    return check_launch();
}

extern "C" int cgx_all_map_fwd(int P, const float* means3D, const float* scales, const float* rotations,
                               const int32_t* radii, const float* viewmatrix, const float* campos, float* all_map,
                               void* stream)
{
    if (P < 0) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means3D || !scales || !rotations || !viewmatrix || !campos || !all_map || !aligned16(rotations))
        return CGX_EINVAL;
    all_map_kernel<<<(P + 255) / 256, 256, 0, (cudaStream_t)stream>>>(P, means3D, scales, (const float4*)rotations,
                                                                      radii, viewmatrix, campos, all_map);
    return check_launch();
}

extern "C" int cgx_all_map_bwd(int P, const float* means3D, const float* scales, const float* rotations,
                               const int32_t* radii, const float* viewmatrix, const float* campos,
                               const float* dL_dall_map, float* dL_dmeans3D, float* dL_drotations, void* stream)
{
    if (P < 0) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!means3D || !scales || !rotations || !viewmatrix || !campos || !dL_dall_map || !dL_dmeans3D ||
        !dL_drotations || !aligned16(rotations) || !aligned16(dL_drotations))
        return CGX_EINVAL;
    all_map_bwd_kernel<<<(P + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        P, means3D, scales, (const float4*)rotations, radii, viewmatrix, campos, dL_dall_map, dL_dmeans3D,
        (float4*)dL_drotations);
    return check_launch();
}

static int fill_cams(CamBatch& cb, int B, const cgx_camera* cams)
{
    if (B <= 0 || B > MAX_CAMS || !cams) return CGX_EINVAL;
    cb.B = B;
    for (int b = 0; b < B; b++) {
        if (!cams[b].viewmatrix || !cams[b].projmatrix || cams[b].W <= 0 || cams[b].H <= 0) return CGX_EINVAL;
        cb.view[b] = cams[b].viewmatrix;
        cb.proj[b] = cams[b].projmatrix;
        cb.tan_fovx[b] = cams[b].tanfovx;
        cb.tan_fovy[b] = cams[b].tanfovy;
        cb.focal_y[b] = cams[b].H / (2.0f * cams[b].tanfovy);
        cb.focal_x[b] = cams[b].W / (2.0f * cams[b].tanfovx);
        cb.W[b] = cams[b].W;
        cb.H[b] = cams[b].H;
    }
    return CGX_OK;
}

extern "C" int cgx_preprocess_fwd_batched_planes(int P, int B, const float* means3D, const float* scales,
                                                 float scale_modifier, const float* rotations,
                                                 const float* opacities, const cgx_camera* cams,
                                                 const float* const* campos, float* const* means2D,
                                                 float* const* depths, int32_t* const* radii,
                                                 float* const* conic_opacity, float* const* all_map, void* stream)
{
    if (P < 0) return CGX_EINVAL;
    CamBatch cb;
    int st = fill_cams(cb, B, cams);
    if (st != CGX_OK) return st;
    if (P == 0) return CGX_OK;
    if (!means3D || !scales || !rotations || !opacities || !means2D || !depths || !radii || !conic_opacity)
        return CGX_EINVAL;
    if ((all_map != nullptr) != (campos != nullptr)) return CGX_EINVAL;
    CamOutputs o;
    CamPlanes pl;
    memset(&pl, 0, sizeof(pl));
    for (int b = 0; b < B; b++) {
        if (!means2D[b] || !depths[b] || !radii[b] || !conic_opacity[b]) return CGX_EINVAL;
        if (((uintptr_t)means2D[b] & 7) || !aligned16(conic_opacity[b])) return CGX_EINVAL;
        o.means2D[b] = (float2*)means2D[b];
        o.depths[b] = depths[b];
        o.radii[b] = radii[b];
        o.conic_opacity[b] = (float4*)conic_opacity[b];
        if (all_map && all_map[b]) {
            if (!campos[b]) return CGX_EINVAL;
            pl.all_map[b] = all_map[b];
            pl.campos[b] = campos[b];
        }
    }
    const int vec_mask = (aligned16(means3D) ? 1 : 0) | (aligned16(scales) ? 2 : 0) | (aligned16(rotations) ? 4 : 0);
    preprocess_fwd_batched_kernel<<<(P + CGX_BLOCK_SIZE - 1) / CGX_BLOCK_SIZE, CGX_BLOCK_SIZE, 0,
                                    (cudaStream_t)stream>>>(P, means3D, scales, scale_modifier, rotations, opacities, cb,
                                                            o, pl, vec_mask);
    return check_launch();
}

extern "C" int cgx_preprocess_fwd_batched(int P, int B, const float* means3D, const float* scales,
                                          float scale_modifier, const float* rotations, const float* opacities,
                                          const cgx_camera* cams, float* const* means2D, float* const* depths,
                                          int32_t* const* radii, float* const* conic_opacity, void* stream)
{
    return cgx_preprocess_fwd_batched_planes(P, B, means3D, scales, scale_modifier, rotations, opacities, cams, nullptr,
                                             means2D, depths, radii, conic_opacity, nullptr, stream);
}

extern "C" int cgx_preprocess_bwd_batched_planes(int P, int B, const float* means3D, const float* scales,
                                                 float scale_modifier, const float* rotations, const cgx_camera* cams,
                                                 const float* const* campos, const int32_t* const* radii,
                                                 const float* const* dL_dmeans2D,
                                                 const float* const* dL_dconic_opacity,
                                                 const float* const* dL_dall_map, float* dL_dmeans3D,
                                                 float* dL_dscales, float* dL_drotations, float* dL_dopacity,
                                                 void* stream)
{
    if (P < 0) return CGX_EINVAL;
    CamBatch cb;
    int st = fill_cams(cb, B, cams);
    if (st != CGX_OK) return st;
    if (P == 0) return CGX_OK;
    if (!means3D || !scales || !rotations || !radii || !dL_dmeans2D || !dL_dconic_opacity || !dL_dmeans3D ||
        !dL_dscales || !dL_drotations || !dL_dopacity || !aligned16(dL_drotations))
        return CGX_EINVAL;
    if ((dL_dall_map != nullptr) != (campos != nullptr)) return CGX_EINVAL;
    CamCotangents c;
    CamPlanes pl;
    memset(&pl, 0, sizeof(pl));
    for (int b = 0; b < B; b++) {
        if (!radii[b] || !dL_dmeans2D[b] || !dL_dconic_opacity[b]) return CGX_EINVAL;
        if (((uintptr_t)dL_dmeans2D[b] & 7) || !aligned16(dL_dconic_opacity[b])) return CGX_EINVAL;
        c.radii[b] = radii[b];
        c.dL_dmeans2D[b] = (const float2*)dL_dmeans2D[b];
        c.dL_dconic_opacity[b] = (const float4*)dL_dconic_opacity[b];
        if (dL_dall_map && dL_dall_map[b]) {
            if (!campos[b]) return CGX_EINVAL;
            pl.dL_dall_map[b] = dL_dall_map[b];
            pl.campos[b] = campos[b];
        }
    }
    const int vec_mask = (aligned16(means3D) ? 1 : 0) | (aligned16(scales) ? 2 : 0) | (aligned16(rotations) ? 4 : 0) |
                         (aligned16(dL_dmeans3D) ? 8 : 0) | (aligned16(dL_dscales) ? 16 : 0);
#if CGX_PRE_BWD_COMPACT
    preprocess_bwd_batched_compact_kernel<<<(P + CGX_BLOCK_SIZE - 1) / CGX_BLOCK_SIZE, CGX_BLOCK_SIZE, 0,
                                            (cudaStream_t)stream>>>(P, means3D, scales, scale_modifier, rotations, cb,
                                                                    c, pl, dL_dmeans3D, dL_dscales,
                                                                    (float4*)dL_drotations, dL_dopacity, vec_mask);
#else
    preprocess_bwd_batched_kernel<<<(P + CGX_BLOCK_SIZE - 1) / CGX_BLOCK_SIZE, CGX_BLOCK_SIZE, 0,
                                    (cudaStream_t)stream>>>(P, means3D, scales, scale_modifier, rotations, cb, c, pl,
                                                            dL_dmeans3D, dL_dscales, (float4*)dL_drotations,
                                                            dL_dopacity, vec_mask);
#endif
    return check_launch();
}

extern "C" int cgx_preprocess_bwd_batched(int P, int B, const float* means3D, const float* scales,
                                          float scale_modifier, const float* rotations, const cgx_camera* cams,
                                          const int32_t* const* radii, const float* const* dL_dmeans2D,
                                          const float* const* dL_dconic_opacity, float* dL_dmeans3D, float* dL_dscales,
                                          float* dL_drotations, float* dL_dopacity, void* stream)
{
    return cgx_preprocess_bwd_batched_planes(P, B, means3D, scales, scale_modifier, rotations, cams, nullptr, radii,
                                             dL_dmeans2D, dL_dconic_opacity, nullptr, dL_dmeans3D, dL_dscales,
                                             dL_drotations, dL_dopacity, stream);
}

extern "C" size_t cgx_preprocess_bwd_rows_workspace_bytes(int P) { return (size_t)(P > 0 ? P : 0) * ROW_ACC * sizeof(float); }

extern "C" int cgx_preprocess_bwd_rows(int P, int n_segments, const cgx_row_segment* segments, int ncols,
                                       const float* rows, const int32_t* row_gaussian, const float* means3D,
                                       const float* scales, float scale_modifier, const float* rotations, int B,
                                       const cgx_camera* cams, const float* const* campos, void* workspace,
                                       size_t workspace_bytes, float* dL_dmeans3D, float* dL_dscales,
                                       float* dL_drotations, float* dL_dopacity, void* stream)
{
    if (P < 0 || n_segments < 0 || n_segments > MAX_ROW_SEGS || (ncols != 14 && ncols != 9)) return CGX_EINVAL;
    CamBatch cb;
    int st = fill_cams(cb, B, cams);
    if (st != CGX_OK) return st;
    if (P == 0) return CGX_OK;
    if (!means3D || !scales || !rotations || !dL_dmeans3D || !dL_dscales || !dL_drotations || !dL_dopacity ||
        !workspace || !aligned16(workspace) || !aligned16(rotations) || !aligned16(dL_drotations))
        return CGX_EINVAL;
    if (workspace_bytes < cgx_preprocess_bwd_rows_workspace_bytes(P)) return CGX_ENOMEM;
    if (n_segments && (!segments || !rows || !row_gaussian)) return CGX_EINVAL;
    RowSegments sg;
    memset(&sg, 0, sizeof(sg));
    CamPlanes pl;
    memset(&pl, 0, sizeof(pl));
    int longest = 0;
    for (int k = 0; k < n_segments; k++) {
        const cgx_row_segment& e = segments[k];
        if (e.start < 0 || e.count < 0 || e.count > 0x7fffffffLL || e.camera < 0 || e.camera >= B) return CGX_EINVAL;
        sg.start[k] = e.start;
        sg.count[k] = (int)e.count;
        sg.cam[k] = e.camera;
        if ((int)e.count > longest) longest = (int)e.count;
    }
    if (ncols == 14) {
        if (!campos) return CGX_EINVAL;
        for (int b = 0; b < B; b++) {
            if (!campos[b]) return CGX_EINVAL;
            pl.campos[b] = campos[b];
        }
    }
    cudaStream_t cs = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(workspace, 0, cgx_preprocess_bwd_rows_workspace_bytes(P), cs);
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    int launched = 0;
    if (longest > 0) {
        const dim3 grid((unsigned)((longest + 255) / 256), (unsigned)n_segments);
        if (ncols == 14)
            preprocess_bwd_rows_kernel<14><<<grid, 256, 0, cs>>>(sg, rows, row_gaussian, means3D, scales, scale_modifier,
                                                                 (const float4*)rotations, cb, pl, (float*)workspace);
        else
            preprocess_bwd_rows_kernel<9><<<grid, 256, 0, cs>>>(sg, rows, row_gaussian, means3D, scales, scale_modifier,
                                                                (const float4*)rotations, cb, pl, (float*)workspace);
        launched++;
    }
    preprocess_bwd_rows_finish_kernel<<<(P + 255) / 256, 256, 0, cs>>>(P, scales, scale_modifier,
                                                                       (const float4*)rotations,
                                                                       (const float*)workspace, dL_dmeans3D, dL_dscales,
                                                                       (float4*)dL_drotations, dL_dopacity);
    return check_launch(launched + 1);
}
