/*
 * CPU oracle for the CityGS-X rasterizer hot path.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls this file.  Only tests,
 * the smoke check and the benchmark's cpu_baseline / reference legs use it.
 *
 * Every function restates, in plain sequential C, what one kernel of the
 * reference CUDA rasterizer computes (paths below are relative to the
 * reference project, RAST = submodule_cityx/diff-gaussian-rasterization):
 *   orc_preprocess_fwd    RAST/cuda_rasterizer/forward.cu:119-153,75-114,183-258
 *                         RAST/cuda_rasterizer/auxiliary.h:52-76,112-131,193-218
 *   orc_filter_preprocess RAST/cuda_rasterizer/forward.cu:545-620
 *   orc_mark_visible      RAST/cuda_rasterizer/rasterizer_impl.cu:58-70
 *   orc_local2j_mask      RAST/rasterize_points.cu:445-492
 *   orc_tile_count        RAST/cuda_rasterizer/rasterizer_impl.cu:264-288 (+ inclusive scan :648)
 *   orc_emit_keys         RAST/cuda_rasterizer/rasterizer_impl.cu:74-117
 *   orc_sort_pairs        stable ascending sort on key bits [0, 32+bit) (:39-54, :675-684)
 *   orc_tile_ranges       RAST/cuda_rasterizer/rasterizer_impl.cu:122-144, :687
 *   orc_render_fwd        RAST/cuda_rasterizer/forward.cu:264-437
 *   orc_tile_stats        RAST/cuda_rasterizer/rasterizer_impl.cu:219-262
 *   orc_render_bwd        RAST/cuda_rasterizer/backward.cu:324-567
 *   orc_preprocess_bwd    RAST/cuda_rasterizer/backward.cu:69-199,203-266,271-321
 *                         RAST/rasterize_points.cu:181-194
 *   orc_sh_to_rgb         RAST/cuda_rasterizer/forward.cu:21-72 (present but unused upstream)
 *
 * Parity status: the reference ships no tests or golden vectors for this
 * path.  The oracle is pinned against outputs of the reference's own CUDA
 * extension (captured on a B200, stored under tests/golden/).  Floating
 * point here is fp32 without fused multiply-add contraction (build with
 * -ffp-contract=off); the GPU contracts, so integer outputs derived from
 * floats (radii, tile rectangles) can differ on inputs that sit within
 * rounding distance of an integer boundary.  orc_preprocess_fwd reports
 * those inputs in `fragile` so tests compare the rest exactly.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define BLOCK_X 16
#define BLOCK_Y 16
#define BLOCK_SIZE 256
#define NCH 3
#define NMAP 5

static inline int imin(int a, int b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }

/* 3x3 matrices are stored the way the reference's math library stores them:
 * m[c][r], column-major, constructor arguments fill columns in order.      */
typedef struct { float m[3][3]; } mat3;

static mat3 mat3_mul(const mat3 *a, const mat3 *b)
{
    mat3 r;
    for (int c = 0; c < 3; c++)
        for (int row = 0; row < 3; row++)
            r.m[c][row] = a->m[0][row] * b->m[c][0] + a->m[1][row] * b->m[c][1] + a->m[2][row] * b->m[c][2];
    return r;
}

static mat3 mat3_t(const mat3 *a)
{
    mat3 r;
    for (int c = 0; c < 3; c++)
        for (int row = 0; row < 3; row++)
            r.m[c][row] = a->m[row][c];
    return r;
}

static inline float ndc2pix(float v, int S) { return (float)((((double)v + 1.0) * (double)S - 1.0) * 0.5); }

/* auxiliary.h:66-76.  Arithmetic is float; truncation toward zero. */
static void get_rect(float px, float py, int r, int gx, int gy, int *x0, int *y0, int *x1, int *y1)
{
    *x0 = imin(gx, imax(0, (int)((px - (float)r) / (float)BLOCK_X)));
    *y0 = imin(gy, imax(0, (int)((py - (float)r) / (float)BLOCK_Y)));
    *x1 = imin(gx, imax(0, (int)((px + (float)r + (float)BLOCK_X - (float)1) / (float)BLOCK_X)));
    *y1 = imin(gy, imax(0, (int)((py + (float)r + (float)BLOCK_Y - (float)1) / (float)BLOCK_Y)));
}

static void xform4x3(const float *p, const float *M, float *o)
{
    o[0] = M[0] * p[0] + M[4] * p[1] + M[8] * p[2] + M[12];
    o[1] = M[1] * p[0] + M[5] * p[1] + M[9] * p[2] + M[13];
    o[2] = M[2] * p[0] + M[6] * p[1] + M[10] * p[2] + M[14];
}

static void xform4x4(const float *p, const float *M, float *o)
{
    o[0] = M[0] * p[0] + M[4] * p[1] + M[8] * p[2] + M[12];
    o[1] = M[1] * p[0] + M[5] * p[1] + M[9] * p[2] + M[13];
    o[2] = M[2] * p[0] + M[6] * p[1] + M[10] * p[2] + M[14];
    o[3] = M[3] * p[0] + M[7] * p[1] + M[11] * p[2] + M[15];
}

static mat3 quat_to_R(const float *q)
{
    float r = q[0], x = q[1], y = q[2], z = q[3];
    mat3 R;
    R.m[0][0] = 1.f - 2.f * (y * y + z * z); R.m[0][1] = 2.f * (x * y - r * z); R.m[0][2] = 2.f * (x * z + r * y);
    R.m[1][0] = 2.f * (x * y + r * z); R.m[1][1] = 1.f - 2.f * (x * x + z * z); R.m[1][2] = 2.f * (y * z - r * x);
    R.m[2][0] = 2.f * (x * z - r * y); R.m[2][1] = 2.f * (y * z + r * x); R.m[2][2] = 1.f - 2.f * (x * x + y * y);
    return R;
}

static void cov3d_from_scale_rot(const float *s, float mod, const float *q, float *cov)
{
    mat3 S; memset(&S, 0, sizeof S);
    S.m[0][0] = mod * s[0]; S.m[1][1] = mod * s[1]; S.m[2][2] = mod * s[2];
    mat3 R = quat_to_R(q);          /* quaternion deliberately not normalised */
    mat3 M = mat3_mul(&S, &R);
    mat3 Mt = mat3_t(&M);
    mat3 Sg = mat3_mul(&Mt, &M);
    cov[0] = Sg.m[0][0]; cov[1] = Sg.m[0][1]; cov[2] = Sg.m[0][2];
    cov[3] = Sg.m[1][1]; cov[4] = Sg.m[1][2]; cov[5] = Sg.m[2][2];
}

/* forward.cu:75-114.  Also returns T = W*J for the backward. */
static void cov2d(const float *mean, float fx, float fy, float tanx, float tany, const float *c3, const float *V,
                  float *cov, mat3 *Tout, float *t_out, float *txtz_o, float *tytz_o)
{
    float t[3];
    xform4x3(mean, V, t);
    const float limx = 1.3f * tanx, limy = 1.3f * tany;
    const float txtz = t[0] / t[2], tytz = t[1] / t[2];
    t[0] = fminf(limx, fmaxf(-limx, txtz)) * t[2];
    t[1] = fminf(limy, fmaxf(-limy, tytz)) * t[2];
    mat3 J;
    J.m[0][0] = fx / t[2]; J.m[0][1] = 0.f; J.m[0][2] = -(fx * t[0]) / (t[2] * t[2]);
    J.m[1][0] = 0.f; J.m[1][1] = fy / t[2]; J.m[1][2] = -(fy * t[1]) / (t[2] * t[2]);
    J.m[2][0] = 0.f; J.m[2][1] = 0.f; J.m[2][2] = 0.f;
    mat3 Wm;
    Wm.m[0][0] = V[0]; Wm.m[0][1] = V[4]; Wm.m[0][2] = V[8];
    Wm.m[1][0] = V[1]; Wm.m[1][1] = V[5]; Wm.m[1][2] = V[9];
    Wm.m[2][0] = V[2]; Wm.m[2][1] = V[6]; Wm.m[2][2] = V[10];
    mat3 T = mat3_mul(&Wm, &J);
    mat3 Vrk;
    Vrk.m[0][0] = c3[0]; Vrk.m[0][1] = c3[1]; Vrk.m[0][2] = c3[2];
    Vrk.m[1][0] = c3[1]; Vrk.m[1][1] = c3[3]; Vrk.m[1][2] = c3[4];
    Vrk.m[2][0] = c3[2]; Vrk.m[2][1] = c3[4]; Vrk.m[2][2] = c3[5];
    mat3 Tt = mat3_t(&T), Vt = mat3_t(&Vrk);
    mat3 A = mat3_mul(&Tt, &Vt);
    mat3 C = mat3_mul(&A, &T);
    cov[0] = C.m[0][0] + 0.3f; cov[1] = C.m[0][1]; cov[2] = C.m[1][1] + 0.3f;
    if (Tout) *Tout = T;
    if (t_out) { t_out[0] = t[0]; t_out[1] = t[1]; t_out[2] = t[2]; }
    if (txtz_o) *txtz_o = txtz;
    if (tytz_o) *tytz_o = tytz;
}

static int near_int(float v, float tol)
{
    float r = v - floorf(v);
    float scale = fmaxf(1.0f, fabsf(v));
    return r < tol * scale || (1.0f - r) < tol * scale;
}

/* Shared geometry of preprocess / filter.  Returns radius (0 when culled). */
static int geom_one(const float *p, const float *s, float mod, const float *q, const float *V, const float *Pm,
                    int W, int H, float tanx, float tany, float fx, float fy,
                    float *m2d, float *depth, float *cov3, float *conic, uint8_t *fragile)
{
    const int gx = (W + BLOCK_X - 1) / BLOCK_X, gy = (H + BLOCK_Y - 1) / BLOCK_Y;
    float ph[4], pv[3];
    xform4x4(p, Pm, ph);
    float pw = 1.0f / (ph[3] + 0.0000001f);
    float projx = ph[0] * pw, projy = ph[1] * pw;
    xform4x3(p, V, pv);
    if (fragile) *fragile = 0;
    if (pv[2] <= 0.0f) { if (fragile && fabsf(pv[2]) < 1e-4f) *fragile = 1; return 0; }
    float c3[6];
    cov3d_from_scale_rot(s, mod, q, c3);
    if (cov3) memcpy(cov3, c3, sizeof c3);
    float cov[3];
    cov2d(p, fx, fy, tanx, tany, c3, V, cov, NULL, NULL, NULL, NULL);
    float det = cov[0] * cov[2] - cov[1] * cov[1];
    if (det == 0.0f) return 0;
    float det_inv = 1.f / det;
    float mid = 0.5f * (cov[0] + cov[2]);
    float l1 = mid + sqrtf(fmaxf(0.1f, mid * mid - det));
    float l2 = mid - sqrtf(fmaxf(0.1f, mid * mid - det));
    float pre = 3.f * sqrtf(fmaxf(l1, l2));
    float my_radius = ceilf(pre);
    float px = ndc2pix(projx, W), py = ndc2pix(projy, H);
    int x0, y0, x1, y1;
    get_rect(px, py, (int)my_radius, gx, gy, &x0, &y0, &x1, &y1);
    if (fragile) {
        float r = (float)(int)my_radius;
        if (near_int(pre, 2e-5f) ||
            near_int((px - r) / 16.f, 2e-5f) || near_int((py - r) / 16.f, 2e-5f) ||
            near_int((px + r + 15.f) / 16.f, 2e-5f) || near_int((py + r + 15.f) / 16.f, 2e-5f))
            *fragile = 1;
    }
    if ((unsigned)(x1 - x0) * (unsigned)(y1 - y0) == 0) return 0;
    if (m2d) { m2d[0] = px; m2d[1] = py; }
    if (depth) *depth = pv[2];
    if (conic) { conic[0] = cov[2] * det_inv; conic[1] = -cov[1] * det_inv; conic[2] = cov[0] * det_inv; }
    return (int)my_radius;
}

/* Outputs must be zero-filled by the caller (the reference allocates them with torch::full(0)). */
void orc_preprocess_fwd(int P, const float *means3D, const float *scales, float mod, const float *rot,
                        const float *opac, const float *V, const float *Pm, int W, int H, float tanx, float tany,
                        float *means2D, float *depths, int *radii, float *cov3D, float *conic_opacity,
                        uint8_t *fragile)
{
    const float fy = H / (2.0f * tany), fx = W / (2.0f * tanx);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < P; i++) {
        float m2[2] = {0, 0}, d = 0, con[3] = {0, 0, 0};
        int r = geom_one(means3D + 3 * i, scales + 3 * i, mod, rot + 4 * i, V, Pm, W, H, tanx, tany, fx, fy,
                         m2, &d, cov3D + 6 * i, con, fragile ? fragile + i : NULL);
        radii[i] = r;
        if (r > 0) {
            means2D[2 * i] = m2[0]; means2D[2 * i + 1] = m2[1];
            depths[i] = d;
            conic_opacity[4 * i] = con[0]; conic_opacity[4 * i + 1] = con[1];
            conic_opacity[4 * i + 2] = con[2]; conic_opacity[4 * i + 3] = opac[i];
        }
    }
}

void orc_filter_preprocess(int P, const float *means3D, const float *scales, float mod, const float *rot,
                           const float *V, const float *Pm, int W, int H, float tanx, float tany, int *radii)
{
    const float fy = H / (2.0f * tany), fx = W / (2.0f * tanx);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < P; i++)
        radii[i] = geom_one(means3D + 3 * i, scales + 3 * i, mod, rot + 4 * i, V, Pm, W, H, tanx, tany, fx, fy,
                            NULL, NULL, NULL, NULL, NULL);
}

void orc_mark_visible(int P, const float *means3D, const float *V, uint8_t *present)
{
    for (int i = 0; i < P; i++) {
        float pv[3];
        xform4x3(means3D + 3 * i, V, pv);
        present[i] = pv[2] > 0.0f;
    }
}

/* rasterize_points.cu:445-492; mask must be zero-filled. */
void orc_local2j_mask(int P, int H, int W, int ws, const float *means2D, const int *radii, const int *tile_bounds,
                      int avoid_pixel_all2all, uint8_t *mask)
{
    const int gx = (W + BLOCK_X - 1) / BLOCK_X, gy = (H + BLOCK_Y - 1) / BLOCK_Y;
    for (int i = 0; i < P; i++) {
        int x0, y0, x1, y1;
        get_rect(means2D[2 * i], means2D[2 * i + 1], radii[i], gx, gy, &x0, &y0, &x1, &y1);
        int tmin = y0 * gx + x0, tmax = (y1 - 1) * gx + x1 - 1;
        if (tmax < tmin) continue;
        for (int rk = 0; rk < ws; rk++) {
            int l = tile_bounds[rk], r = tile_bounds[rk + 1];
            if (avoid_pixel_all2all) { l -= gx + 1; r += gx + 1; }
            if (tmax < l || tmin >= r) continue;
            mask[(size_t)i * ws + rk] = 1;
        }
    }
}

/* rasterizer_impl.cu:264-288 followed by the inclusive sum (:648). Returns R. */
int64_t orc_tile_count(int P, int W, int H, const int *radii, const float *means2D, const uint8_t *local,
                       uint32_t *tiles_touched, uint32_t *offsets)
{
    const int gx = (W + BLOCK_X - 1) / BLOCK_X, gy = (H + BLOCK_Y - 1) / BLOCK_Y;
    uint32_t run = 0;
    for (int i = 0; i < P; i++) {
        uint32_t cnt = 0;
        if (radii[i] > 0) {
            int x0, y0, x1, y1;
            get_rect(means2D[2 * i], means2D[2 * i + 1], radii[i], gx, gy, &x0, &y0, &x1, &y1);
            for (int y = y0; y < y1; y++)
                for (int x = x0; x < x1; x++)
                    if (local[y * gx + x]) cnt++;
        }
        tiles_touched[i] = cnt;
        run += cnt;
        offsets[i] = run;
    }
    return (int64_t)run;
}

void orc_emit_keys(int P, int W, int H, const int *radii, const float *means2D, const float *depths,
                   const uint32_t *offsets, const uint8_t *local, uint64_t *keys, uint32_t *vals)
{
    const int gx = (W + BLOCK_X - 1) / BLOCK_X, gy = (H + BLOCK_Y - 1) / BLOCK_Y;
    for (int i = 0; i < P; i++) {
        if (radii[i] <= 0) continue;
        uint32_t off = i == 0 ? 0 : offsets[i - 1];
        int x0, y0, x1, y1;
        get_rect(means2D[2 * i], means2D[2 * i + 1], radii[i], gx, gy, &x0, &y0, &x1, &y1);
        uint32_t dbits;
        memcpy(&dbits, depths + i, 4);
        for (int y = y0; y < y1; y++)
            for (int x = x0; x < x1; x++)
                if (local[y * gx + x]) {
                    keys[off] = ((uint64_t)(uint32_t)(y * gx + x) << 32) | dbits;
                    vals[off] = (uint32_t)i;
                    off++;
                }
    }
}

/* rasterizer_impl.cu:39-54 */
uint32_t orc_higher_msb(uint32_t n)
{
    uint32_t msb = sizeof(n) * 4, step = msb;
    while (step > 1) {
        step /= 2;
        if (n >> msb) msb += step; else msb -= step;
    }
    if (n >> msb) msb++;
    return msb;
}

/* Stable LSD radix sort on bits [0, end_bit).  Bits at and above end_bit do
 * not take part in the comparison but travel with the key. */
void orc_sort_pairs(int64_t n, int end_bit, const uint64_t *kin, const uint32_t *vin, uint64_t *kout, uint32_t *vout)
{
    if (n <= 0) return;
    uint64_t *ka = (uint64_t *)malloc(n * 8), *kb = (uint64_t *)malloc(n * 8);
    uint32_t *va = (uint32_t *)malloc(n * 4), *vb = (uint32_t *)malloc(n * 4);
    memcpy(ka, kin, n * 8); memcpy(va, vin, n * 4);
    for (int shift = 0; shift < end_bit; shift += 8) {
        int bits = imin(8, end_bit - shift);
        uint32_t mask = (1u << bits) - 1;
        int64_t cnt[257]; memset(cnt, 0, sizeof cnt);
        for (int64_t i = 0; i < n; i++) cnt[((ka[i] >> shift) & mask) + 1]++;
        for (int d = 0; d < 256; d++) cnt[d + 1] += cnt[d];
        for (int64_t i = 0; i < n; i++) {
            int64_t dst = cnt[(ka[i] >> shift) & mask]++;
            kb[dst] = ka[i]; vb[dst] = va[i];
        }
        uint64_t *tk = ka; ka = kb; kb = tk;
        uint32_t *tv = va; va = vb; vb = tv;
    }
    memcpy(kout, ka, n * 8); memcpy(vout, va, n * 4);
    free(ka); free(kb); free(va); free(vb);
}

/* ranges is uint2[T], zero-filled here (the reference memsets it). */
void orc_tile_ranges(int64_t L, int T, const uint64_t *keys, uint32_t *ranges)
{
    memset(ranges, 0, (size_t)T * 8);
    for (int64_t i = 0; i < L; i++) {
        uint32_t cur = (uint32_t)(keys[i] >> 32);
        if (i == 0) ranges[2 * cur] = 0;
        else {
            uint32_t prev = (uint32_t)(keys[i - 1] >> 32);
            if (cur != prev) { ranges[2 * prev + 1] = (uint32_t)i; ranges[2 * cur] = (uint32_t)i; }
        }
        if (i == L - 1) ranges[2 * cur + 1] = (uint32_t)L;
    }
}

/* forward.cu:264-437.  Image outputs must be zero-filled (non-local tiles stay 0).
 * out_observe (P ints) must be zero-filled. */
void orc_render_fwd(int W, int H, float tanx, float tany, const uint32_t *ranges, const uint32_t *point_list,
                    const float *means2D, const float *rgb, const float *all_map, const float *conic_opacity,
                    const uint8_t *local, const float *bg, int render_geo,
                    float *final_T, uint32_t *n_contrib, uint32_t *n_contrib2loss,
                    float *out_color, int *out_observe, float *out_all_map, float *out_plane_depth)
{
    const int gx = (W + BLOCK_X - 1) / BLOCK_X, gy = (H + BLOCK_Y - 1) / BLOCK_Y;
    const float fy = H / (2.0f * tany), fx = W / (2.0f * tanx);
    const float cx = (float)(W * 0.5f), cy = (float)(H * 0.5f);
    const size_t HW = (size_t)H * W;
#pragma omp parallel for schedule(dynamic, 4)
    for (int tile = 0; tile < gx * gy; tile++) {
        if (!local[tile]) continue;
        const int tx = tile % gx, ty = tile / gx;
        const uint32_t r0 = ranges[2 * tile], r1 = ranges[2 * tile + 1];
        for (int ly = 0; ly < BLOCK_Y; ly++)
            for (int lx = 0; lx < BLOCK_X; lx++) {
                const int pxi = tx * BLOCK_X + lx, pyi = ty * BLOCK_Y + ly;
                if (pxi >= W || pyi >= H) continue;
                const size_t pix = (size_t)W * pyi + pxi;
                const float pfx = (float)pxi, pfy = (float)pyi;
                const float rayx = (pfx - cx) / fx, rayy = (pfy - cy) / fy;
                float T = 1.0f, C[NCH] = {0}, A[NMAP] = {0};
                uint32_t contributor = 0, last = 0, c2l = 0;
                for (uint32_t k = r0; k < r1; k++) {
                    const uint32_t g = point_list[k];
                    contributor++;
                    const float dx = means2D[2 * g] - pfx, dy = means2D[2 * g + 1] - pfy;
                    const float *co = conic_opacity + 4 * (size_t)g;
                    const float power = -0.5f * (co[0] * dx * dx + co[2] * dy * dy) - co[1] * dx * dy;
                    if (power > 0.0f) continue;
                    const float alpha = fminf(0.99f, co[3] * expf(power));
                    if (alpha < 1.0f / 255.0f) continue;
                    const float test_T = T * (1 - alpha);
                    if (test_T < 0.0001f) break;       /* pixel done; contributor was counted */
                    c2l++;
                    for (int ch = 0; ch < NCH; ch++) C[ch] += rgb[(size_t)g * NCH + ch] * alpha * T;
                    if (render_geo)
                        for (int ch = 0; ch < NMAP; ch++) A[ch] += all_map[(size_t)g * NMAP + ch] * alpha * T;
                    if (T > 0.5f) {
#pragma omp atomic
                        out_observe[g] += 1;
                    }
                    T = test_T;
                    last = contributor;
                }
                final_T[pix] = T;
                n_contrib[pix] = last;
                n_contrib2loss[pix] = c2l;
                for (int ch = 0; ch < NCH; ch++) out_color[ch * HW + pix] = C[ch] + T * bg[ch];
                if (render_geo) {
                    for (int ch = 0; ch < NMAP; ch++) out_all_map[ch * HW + pix] = A[ch];
                    out_plane_depth[pix] =
                        (float)((double)A[4] / -((double)(A[0] * rayx + A[1] * rayy + A[2]) + 1.0e-8));
                }
            }
    }
}

/* rasterizer_impl.cu:219-262: per-tile range length and per-tile sums of the
 * two per-pixel counters.  Non-local tiles keep 0 in the two sums. */
void orc_tile_stats(int W, int H, const uint32_t *ranges, const uint32_t *n_contrib_px, const uint32_t *n_c2l_px,
                    const uint8_t *local, int *n_render, int *n_consider, int *n_contrib)
{
    const int gx = (W + BLOCK_X - 1) / BLOCK_X, gy = (H + BLOCK_Y - 1) / BLOCK_Y;
    for (int tile = 0; tile < gx * gy; tile++) {
        n_render[tile] = (int)(ranges[2 * tile + 1] - ranges[2 * tile]);
        if (!local[tile]) continue;
        const int tx = tile % gx, ty = tile / gx;
        int a = 0, b = 0;
        for (int ly = 0; ly < BLOCK_Y; ly++)
            for (int lx = 0; lx < BLOCK_X; lx++) {
                const int pxi = tx * BLOCK_X + lx, pyi = ty * BLOCK_Y + ly;
                if (pxi >= W || pyi >= H) continue;
                a += (int)n_contrib_px[(size_t)W * pyi + pxi];
                b += (int)n_c2l_px[(size_t)W * pyi + pxi];
            }
        n_consider[tile] = a;
        n_contrib[tile] = b;
    }
}

/* Per-Gaussian gradient sums are accumulated in double and narrowed once at the end: the sums cancel heavily
 * and their fp32 value depends on the (unordered) summation order, on the GPU as much as here; the double
 * accumulator makes the oracle the order-independent value both are compared with. */
static inline void atomic_addd(double *p, float v)
{
#pragma omp atomic
    *p += (double)v;
}

/* backward.cu:324-567.  Gradient outputs must be zero-filled:
 * dL_dmean2D (P,3), dL_dmean2D_abs (P,3), dL_dconic (P,4) [= (P,2,2)],
 * dL_dopacity (P), dL_dcolors (P,3), dL_dall_map (P,5). */
void orc_render_bwd(int P, int W, int H, float tanx, float tany, const uint32_t *ranges, const uint32_t *point_list,
                    const float *bg, const float *means2D, const float *conic_opacity, const float *rgb,
                    const float *all_map, const float *all_map_pixels, const float *final_T,
                    const uint32_t *n_contrib, const uint8_t *local, const float *dL_dpix,
                    const float *dL_dout_all_map, const float *dL_dout_plane_depth, int render_geo,
                    float *dL_dmean2D, float *dL_dmean2D_abs, float *dL_dconic, float *dL_dopacity,
                    float *dL_dcolors, float *dL_dall_map)
{
    const int gx = (W + BLOCK_X - 1) / BLOCK_X, gy = (H + BLOCK_Y - 1) / BLOCK_Y;
    const float fy = H / (2.0f * tany), fx = W / (2.0f * tanx);
    const size_t HW = (size_t)H * W;
    const float ddelx_dx = (float)(0.5 * W), ddely_dy = (float)(0.5 * H);
    /* 16 double accumulators per Gaussian: mean2D x,y | abs x,y | conic [0,0],[0,1],[1,1] | opacity | rgb 3 | map 5 */
    double *acc = (double *)calloc((size_t)(P > 0 ? P : 1) * 16, sizeof(double));
#pragma omp parallel for schedule(dynamic, 4)
    for (int tile = 0; tile < gx * gy; tile++) {
        if (!local[tile]) continue;
        const int tx = tile % gx, ty = tile / gx;
        const uint32_t r0 = ranges[2 * tile], r1 = ranges[2 * tile + 1];
        for (int ly = 0; ly < BLOCK_Y; ly++)
            for (int lx = 0; lx < BLOCK_X; lx++) {
                const int pxi = tx * BLOCK_X + lx, pyi = ty * BLOCK_Y + ly;
                if (pxi >= W || pyi >= H) continue;
                const size_t pix = (size_t)W * pyi + pxi;
                const float pfx = (float)pxi, pfy = (float)pyi;
                const float rayx = (float)(((double)pfx - W * 0.5) / (double)fx);
                const float rayy = (float)(((double)pfy - H * 0.5) / (double)fy);
                const float T_final = final_T[pix];
                float T = T_final;
                uint32_t contributor = r1 - r0;
                const uint32_t last_contributor = n_contrib[pix];
                float accum_rec[NCH] = {0}, accum_map[NMAP] = {0};
                float dpix[NCH], dmap[NMAP] = {0};
                for (int i = 0; i < NCH; i++) dpix[i] = dL_dpix[i * HW + pix];
                if (render_geo) {
                    for (int i = 0; i < NMAP; i++) dmap[i] = dL_dout_all_map[i * HW + pix];
                    const float nx = all_map_pixels[pix], ny = all_map_pixels[HW + pix], nz = all_map_pixels[2 * HW + pix];
                    const float distance = all_map_pixels[4 * HW + pix];
                    const float tmp = (float)((double)(nx * rayx + ny * rayy + nz) + 1.0e-8);
                    const float dpd = dL_dout_plane_depth[pix];
                    dmap[NMAP - 1] += (-dpd / tmp);
                    dmap[0] += dpd * (distance / (tmp * tmp) * rayx);
                    dmap[1] += dpd * (distance / (tmp * tmp) * rayy);
                    dmap[2] += dpd * (distance / (tmp * tmp));
                }
                float last_alpha = 0, last_color[NCH] = {0}, last_map[NMAP] = {0};
                for (uint32_t k = r1; k-- > r0;) {
                    contributor--;
                    if (contributor >= last_contributor) continue;
                    const uint32_t g = point_list[k];
                    double *a16 = acc + (size_t)g * 16;
                    const float dx = means2D[2 * g] - pfx, dy = means2D[2 * g + 1] - pfy;
                    const float *co = conic_opacity + 4 * (size_t)g;
                    const float power = -0.5f * (co[0] * dx * dx + co[2] * dy * dy) - co[1] * dx * dy;
                    if (power > 0.0f) continue;
                    const float G = expf(power);
                    const float alpha = fminf(0.99f, co[3] * G);
                    if (alpha < 1.0f / 255.0f) continue;
                    T = T / (1.f - alpha);
                    const float dchannel_dcolor = alpha * T;
                    float dL_dalpha = 0.0f;
                    for (int ch = 0; ch < NCH; ch++) {
                        const float c = rgb[(size_t)g * NCH + ch];
                        accum_rec[ch] = last_alpha * last_color[ch] + (1.f - last_alpha) * accum_rec[ch];
                        last_color[ch] = c;
                        dL_dalpha += (c - accum_rec[ch]) * dpix[ch];
                        atomic_addd(&a16[8 + ch], dchannel_dcolor * dpix[ch]);
                    }
                    if (render_geo)
                        for (int ch = 0; ch < NMAP; ch++) {
                            const float c = all_map[(size_t)g * NMAP + ch];
                            accum_map[ch] = last_alpha * last_map[ch] + (1.f - last_alpha) * accum_map[ch];
                            last_map[ch] = c;
                            dL_dalpha += (c - accum_map[ch]) * dmap[ch];
                            atomic_addd(&a16[11 + ch], dchannel_dcolor * dmap[ch]);
                        }
                    dL_dalpha *= T;
                    last_alpha = alpha;
                    float bg_dot = 0;
                    for (int i = 0; i < NCH; i++) bg_dot += bg[i] * dpix[i];
                    dL_dalpha += (-T_final / (1.f - alpha)) * bg_dot;
                    const float dL_dG = co[3] * dL_dalpha;
                    const float gdx = G * dx, gdy = G * dy;
                    const float dG_ddelx = -gdx * co[0] - gdy * co[1];
                    const float dG_ddely = -gdy * co[2] - gdx * co[1];
                    atomic_addd(&a16[0], dL_dG * dG_ddelx * ddelx_dx);
                    atomic_addd(&a16[1], dL_dG * dG_ddely * ddely_dy);
                    atomic_addd(&a16[2], fabsf(dL_dG * dG_ddelx * ddelx_dx));
                    atomic_addd(&a16[3], fabsf(dL_dG * dG_ddely * ddely_dy));
                    atomic_addd(&a16[4], -0.5f * gdx * dx * dL_dG);
                    atomic_addd(&a16[5], -0.5f * gdx * dy * dL_dG);
                    atomic_addd(&a16[6], -0.5f * gdy * dy * dL_dG);
                    atomic_addd(&a16[7], G * dL_dalpha);
                }
            }
    }
#pragma omp parallel for schedule(static)
    for (int g = 0; g < P; g++) {
        const double *a16 = acc + (size_t)g * 16;
        dL_dmean2D[3 * (size_t)g] = (float)a16[0]; dL_dmean2D[3 * (size_t)g + 1] = (float)a16[1];
        dL_dmean2D_abs[3 * (size_t)g] = (float)a16[2]; dL_dmean2D_abs[3 * (size_t)g + 1] = (float)a16[3];
        dL_dconic[4 * (size_t)g] = (float)a16[4]; dL_dconic[4 * (size_t)g + 1] = (float)a16[5];
        dL_dconic[4 * (size_t)g + 3] = (float)a16[6];
        dL_dopacity[g] = (float)a16[7];
        for (int ch = 0; ch < NCH; ch++) dL_dcolors[(size_t)g * NCH + ch] = (float)a16[8 + ch];
        for (int ch = 0; ch < NMAP; ch++) dL_dall_map[(size_t)g * NMAP + ch] = (float)a16[11 + ch];
    }
    free(acc);
}

/* backward.cu:69-199 + 271-321 + 203-266, with the (P,4) conic_opacity
 * cotangent split as rasterize_points.cu:181-194 does: conic (a,b,c) =
 * columns 0,1,2 land in the (P,2,2) slots [0,0],[0,1],[1,1]; opacity = col 3.
 * dL_dmean2D is (P,2).  Outputs (zero-filled by caller): dL_dmeans3D (P,3),
 * dL_dscales (P,3), dL_drot (P,4), dL_dopacity (P,1). */
void orc_preprocess_bwd(int P, const float *means3D, const float *scales, float mod, const float *rot,
                        const int *radii, const float *cov3Ds, const float *V, const float *Pm, int W, int H,
                        float tanx, float tany, const float *dL_dmean2D, const float *dL_dconic_opacity,
                        float *dL_dmeans3D, float *dL_dscales, float *dL_drot, float *dL_dopacity)
{
    const float fy = H / (2.0f * tany), fx = W / (2.0f * tanx);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < P; i++) {
        dL_dopacity[i] = dL_dconic_opacity[4 * i + 3];
        if (!(radii[i] > 0)) continue;
        const float *mean = means3D + 3 * i;
        const float *c3 = cov3Ds + 6 * i;
        /* --- computeCov2DCUDA --- */
        const float dcx = dL_dconic_opacity[4 * i], dcy = dL_dconic_opacity[4 * i + 1], dcz = dL_dconic_opacity[4 * i + 2];
        float cov[3], t[3], txtz, tytz;
        mat3 T;
        cov2d(mean, fx, fy, tanx, tany, c3, V, cov, &T, t, &txtz, &tytz);
        const float limx = 1.3f * tanx, limy = 1.3f * tany;
        const float x_grad_mul = (txtz < -limx || txtz > limx) ? 0.f : 1.f;
        const float y_grad_mul = (tytz < -limy || tytz > limy) ? 0.f : 1.f;
        const float a = cov[0], b = cov[1], c = cov[2];
        const float denom = a * c - b * b;
        float dL_da = 0, dL_db = 0, dL_dc = 0;
        const float denom2inv = 1.0f / ((denom * denom) + 0.0000001f);
        float dcov[6];
        if (denom2inv != 0) {
            dL_da = denom2inv * (-c * c * dcx + 2 * b * c * dcy + (denom - a * c) * dcz);
            dL_dc = denom2inv * (-a * a * dcz + 2 * a * b * dcy + (denom - a * c) * dcx);
            dL_db = denom2inv * 2 * (b * c * dcx - (denom + 2 * b * b) * dcy + a * b * dcz);
            dcov[0] = (T.m[0][0] * T.m[0][0] * dL_da + T.m[0][0] * T.m[1][0] * dL_db + T.m[1][0] * T.m[1][0] * dL_dc);
            dcov[3] = (T.m[0][1] * T.m[0][1] * dL_da + T.m[0][1] * T.m[1][1] * dL_db + T.m[1][1] * T.m[1][1] * dL_dc);
            dcov[5] = (T.m[0][2] * T.m[0][2] * dL_da + T.m[0][2] * T.m[1][2] * dL_db + T.m[1][2] * T.m[1][2] * dL_dc);
            dcov[1] = 2 * T.m[0][0] * T.m[0][1] * dL_da + (T.m[0][0] * T.m[1][1] + T.m[0][1] * T.m[1][0]) * dL_db + 2 * T.m[1][0] * T.m[1][1] * dL_dc;
            dcov[2] = 2 * T.m[0][0] * T.m[0][2] * dL_da + (T.m[0][0] * T.m[1][2] + T.m[0][2] * T.m[1][0]) * dL_db + 2 * T.m[1][0] * T.m[1][2] * dL_dc;
            dcov[4] = 2 * T.m[0][2] * T.m[0][1] * dL_da + (T.m[0][1] * T.m[1][2] + T.m[0][2] * T.m[1][1]) * dL_db + 2 * T.m[1][1] * T.m[1][2] * dL_dc;
        } else {
            for (int k = 0; k < 6; k++) dcov[k] = 0;
        }
        float Vk[3][3] = {{c3[0], c3[1], c3[2]}, {c3[1], c3[3], c3[4]}, {c3[2], c3[4], c3[5]}};
        float dT[2][3];
        for (int k = 0; k < 3; k++) {
            dT[0][k] = 2 * (T.m[0][0] * Vk[k][0] + T.m[0][1] * Vk[k][1] + T.m[0][2] * Vk[k][2]) * dL_da +
                       (T.m[1][0] * Vk[k][0] + T.m[1][1] * Vk[k][1] + T.m[1][2] * Vk[k][2]) * dL_db;
            dT[1][k] = 2 * (T.m[1][0] * Vk[k][0] + T.m[1][1] * Vk[k][1] + T.m[1][2] * Vk[k][2]) * dL_dc +
                       (T.m[0][0] * Vk[k][0] + T.m[0][1] * Vk[k][1] + T.m[0][2] * Vk[k][2]) * dL_db;
        }
        /* W[c][r] as built in the kernel: W[0]=(V0,V4,V8) W[1]=(V1,V5,V9) W[2]=(V2,V6,V10) */
        const float W00 = V[0], W01 = V[4], W02 = V[8], W10 = V[1], W11 = V[5], W12 = V[9], W20 = V[2], W21 = V[6], W22 = V[10];
        const float dJ00 = W00 * dT[0][0] + W01 * dT[0][1] + W02 * dT[0][2];
        const float dJ02 = W20 * dT[0][0] + W21 * dT[0][1] + W22 * dT[0][2];
        const float dJ11 = W10 * dT[1][0] + W11 * dT[1][1] + W12 * dT[1][2];
        const float dJ12 = W20 * dT[1][0] + W21 * dT[1][1] + W22 * dT[1][2];
        const float tz = 1.f / t[2], tz2 = tz * tz, tz3 = tz2 * tz;
        const float dtx = x_grad_mul * -fx * tz2 * dJ02;
        const float dty = y_grad_mul * -fy * tz2 * dJ12;
        const float dtz = -fx * tz2 * dJ00 - fy * tz2 * dJ11 + (2 * fx * t[0]) * tz3 * dJ02 + (2 * fy * t[1]) * tz3 * dJ12;
        float dmean[3];
        dmean[0] = V[0] * dtx + V[1] * dty + V[2] * dtz;
        dmean[1] = V[4] * dtx + V[5] * dty + V[6] * dtz;
        dmean[2] = V[8] * dtx + V[9] * dty + V[10] * dtz;
        /* --- preprocessCUDA backward --- */
        float mh[4];
        xform4x4(mean, Pm, mh);
        const float m_w = 1.0f / (mh[3] + 0.0000001f);
        const float mul1 = (Pm[0] * mean[0] + Pm[4] * mean[1] + Pm[8] * mean[2] + Pm[12]) * m_w * m_w;
        const float mul2 = (Pm[1] * mean[0] + Pm[5] * mean[1] + Pm[9] * mean[2] + Pm[13]) * m_w * m_w;
        const float gx2 = dL_dmean2D[2 * i], gy2 = dL_dmean2D[2 * i + 1];
        dmean[0] += (Pm[0] * m_w - Pm[3] * mul1) * gx2 + (Pm[1] * m_w - Pm[3] * mul2) * gy2;
        dmean[1] += (Pm[4] * m_w - Pm[7] * mul1) * gx2 + (Pm[5] * m_w - Pm[7] * mul2) * gy2;
        dmean[2] += (Pm[8] * m_w - Pm[11] * mul1) * gx2 + (Pm[9] * m_w - Pm[11] * mul2) * gy2;
        dL_dmeans3D[3 * i] = dmean[0]; dL_dmeans3D[3 * i + 1] = dmean[1]; dL_dmeans3D[3 * i + 2] = dmean[2];
        /* --- computeCov3D backward --- */
        const float *q = rot + 4 * i;
        const float r = q[0], x = q[1], y = q[2], z = q[3];
        mat3 R = quat_to_R(q);
        const float s[3] = {mod * scales[3 * i], mod * scales[3 * i + 1], mod * scales[3 * i + 2]};
        mat3 S; memset(&S, 0, sizeof S);
        S.m[0][0] = s[0]; S.m[1][1] = s[1]; S.m[2][2] = s[2];
        mat3 M = mat3_mul(&S, &R);
        mat3 dSig;
        dSig.m[0][0] = dcov[0]; dSig.m[0][1] = 0.5f * dcov[1]; dSig.m[0][2] = 0.5f * dcov[2];
        dSig.m[1][0] = 0.5f * dcov[1]; dSig.m[1][1] = dcov[3]; dSig.m[1][2] = 0.5f * dcov[4];
        dSig.m[2][0] = 0.5f * dcov[2]; dSig.m[2][1] = 0.5f * dcov[4]; dSig.m[2][2] = dcov[5];
        mat3 M2;
        for (int cc = 0; cc < 3; cc++) for (int rr = 0; rr < 3; rr++) M2.m[cc][rr] = 2.0f * M.m[cc][rr];
        mat3 dM = mat3_mul(&M2, &dSig);
        mat3 Rt = mat3_t(&R), dMt = mat3_t(&dM);
        for (int k = 0; k < 3; k++)
            dL_dscales[3 * i + k] = Rt.m[k][0] * dMt.m[k][0] + Rt.m[k][1] * dMt.m[k][1] + Rt.m[k][2] * dMt.m[k][2];
        for (int k = 0; k < 3; k++) for (int rr = 0; rr < 3; rr++) dMt.m[k][rr] *= s[k];
        float dq[4];
        dq[0] = 2 * z * (dMt.m[0][1] - dMt.m[1][0]) + 2 * y * (dMt.m[2][0] - dMt.m[0][2]) + 2 * x * (dMt.m[1][2] - dMt.m[2][1]);
        dq[1] = 2 * y * (dMt.m[1][0] + dMt.m[0][1]) + 2 * z * (dMt.m[2][0] + dMt.m[0][2]) + 2 * r * (dMt.m[1][2] - dMt.m[2][1]) - 4 * x * (dMt.m[2][2] + dMt.m[1][1]);
        dq[2] = 2 * x * (dMt.m[1][0] + dMt.m[0][1]) + 2 * r * (dMt.m[2][0] - dMt.m[0][2]) + 2 * z * (dMt.m[1][2] + dMt.m[2][1]) - 4 * y * (dMt.m[2][2] + dMt.m[0][0]);
        dq[3] = 2 * r * (dMt.m[0][1] - dMt.m[1][0]) + 2 * x * (dMt.m[2][0] + dMt.m[0][2]) + 2 * y * (dMt.m[1][2] + dMt.m[2][1]) - 4 * z * (dMt.m[1][1] + dMt.m[0][0]);
        for (int k = 0; k < 4; k++) dL_drot[4 * i + k] = dq[k];
    }
}

/* forward.cu:21-72 (degree 0..3); sh is (P, M, 3) with M >= (deg+1)^2. */
void orc_sh_to_rgb(int P, int deg, int M, const float *means3D, const float *campos, const float *sh,
                   float *rgb, uint8_t *clamped)
{
    static const float C0 = 0.28209479177387814f, C1 = 0.4886025119029199f;
    static const float C2[5] = {1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f,
                                -1.0925484305920792f, 0.5462742152960396f};
    static const float C3[7] = {-0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f,
                                -0.4570457994644658f, 1.445305721320277f, -0.5900435899266435f};
#pragma omp parallel for schedule(static)
    for (int i = 0; i < P; i++) {
        float d[3] = {means3D[3 * i] - campos[0], means3D[3 * i + 1] - campos[1], means3D[3 * i + 2] - campos[2]};
        float len = sqrtf(d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
        float x = d[0] / len, y = d[1] / len, z = d[2] / len;
        const float *s = sh + (size_t)i * M * 3;
        for (int ch = 0; ch < 3; ch++) {
#define SH(k) s[(k) * 3 + ch]
            float res = C0 * SH(0);
            if (deg > 0) {
                res = res - C1 * y * SH(1) + C1 * z * SH(2) - C1 * x * SH(3);
                if (deg > 1) {
                    float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
                    res = res + C2[0] * xy * SH(4) + C2[1] * yz * SH(5) + C2[2] * (2.0f * zz - xx - yy) * SH(6) +
                          C2[3] * xz * SH(7) + C2[4] * (xx - yy) * SH(8);
                    if (deg > 2)
                        res = res + C3[0] * y * (3.0f * xx - yy) * SH(9) + C3[1] * xy * z * SH(10) +
                              C3[2] * y * (4.0f * zz - xx - yy) * SH(11) +
                              C3[3] * z * (2.0f * zz - 3.0f * xx - 3.0f * yy) * SH(12) +
                              C3[4] * x * (4.0f * zz - xx - yy) * SH(13) + C3[5] * z * (xx - yy) * SH(14) +
                              C3[6] * x * (xx - 3.0f * yy) * SH(15);
                }
            }
#undef SH
            res += 0.5f;
            clamped[3 * i + ch] = res < 0;
            rgb[3 * i + ch] = res < 0 ? 0.0f : res;
        }
    }
}
