// Per-tile alpha compositing, forward and backward (instruction-issue bound).
//
// One CTA (256 threads, one pixel each) per 16x16 tile, like the reference, but:
//  * the five per-Gaussian inputs are first packed into one 64-byte record per Gaussian
//    [x y | a b c opacity | r g b | m0..m4 | cull extents]; a tile's batch of 256 records is then staged into
//    shared memory by 256 asynchronous 64-byte bulk copies (cp.async.bulk, completion on an mbarrier),
//    double-buffered so the gather of batch i+1 overlaps the blending of batch i;
//  * each warp owns an 8x4 pixel block of the tile and first culls the batch against it with an exact-safe bound
//    (a Gaussian is dropped for the block only if alpha < 1/255 is guaranteed there), 32 Gaussians per ballot;
//  * the survivors ("visits") are processed 32 at a time in two phases.  Phase 1: every lane evaluates alpha of
//    its pixel against each visit and keeps one bit per visit.  Phase 2: every lane walks only its OWN set bits,
//    in list order, so the expensive part (blending; gradient terms in the backward) is executed as often as the
//    busiest pixel of the block contributes, not once per visit: on aerial scenes a visit has 1-5 contributing
//    pixels out of 32;
//  * the backward stages the 16 gradient terms of every contribution in a per-warp shared-memory table (rows
//    grouped by visit through ballot prefix sums), then half-warps sum each visit's rows, one lane per term, and
//    issue ONE atomic per term per Gaussian per warp straight into the caller's gradient tensors (which also
//    performs the (P,2,2)+(P,1) -> (P,4) repack);
//  * the per-tile statistics (sum of per-pixel counters) are reduced in the forward's epilogue.
//
// Every wait on an mbarrier is bounded: when the limit is hit the CTA records an error in the device
// status word, stops blending and returns.
#include "cgx_common.cuh"

#ifndef CGX_EXPERIMENT
#define CGX_EXPERIMENT 0   // timing experiments only: bit 0 skip phase 1, bit 1 skip phase 2, bit 2 skip phase 3,
                           // bit 3 skip the gradient atomics of phase 3
#endif

namespace cgx {

__device__ int g_status = 0;  // 0 ok; CGX_ETIMEDOUT when a bounded wait gave up

constexpr unsigned long long WAIT_LIMIT_CYCLES = 1ull << 31;  // ~1 s at B200 clocks

struct __align__(16) Record {
    float4 q0;  // x, y, conic a, conic b
    float4 q1;  // conic c, opacity, r, g
    float4 q2;  // b, m0, m1, m2
    float4 q3;  // m3, m4, cull half-extent x, cull half-extent y (see cull_extent)
};

// A record as the forward kernel keeps it in shared memory: 80-byte pitch.  In the two-phase walk every lane reads
// the record of a DIFFERENT Gaussian; at the natural 64-byte pitch eight lanes of a quarter-warp would hit the same
// two groups of four banks, at 80 bytes consecutive records fall into all eight groups.
struct __align__(16) RecSlot : Record {
    float4 pad;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false after WAIT_LIMIT_CYCLES without completion.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if ((unsigned long long)(clock64() - t0) > WAIT_LIMIT_CYCLES) return false;
    }
    return true;
}
// 64-byte global -> shared bulk copy, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load_64(void* dst_smem, const void* src_gmem, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 64, [%2];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(smem_u32(bar))
                 : "memory");
}

// Half extents of the axis-aligned box outside of which opacity * exp(power) < 1/255 for certain.
// power = -0.5 (a dx^2 + c dy^2) - b dx dy >= -tau bounds |dx| <= sqrt(2 tau c / (ac - b^2)), same for dy with a.
// The box is inflated (1 % + 0.01 px) so float rounding in the per-pixel test can never keep a pixel the box drops.
__device__ __forceinline__ float2 cull_extent(float a, float b, float c, float o)
{
    const float inf = __int_as_float(0x7f800000);
    if (!(o >= 1.0f / 255.0f)) return {-1.f, -1.f};  // alpha <= o < 1/255 everywhere (NaN opacity: never kept either)
    const float det = a * c - b * b;
    if (!(det > 0.f) || !(a > 0.f) || !(c > 0.f)) return {inf, inf};
    const float tau = __logf(255.0f * o) * 1.01f + 0.01f;
    const float ex = sqrtf(2.f * tau * c / det) * 1.01f + 0.01f;
    const float ey = sqrtf(2.f * tau * a / det) * 1.01f + 0.01f;
    if (!(ex == ex) || !(ey == ey)) return {inf, inf};
    return {ex, ey};
}

// alpha of one Gaussian at one pixel, in the reference's operation order (cuda_rasterizer/forward.cu:376-389).
// Returns false when the pixel is skipped (power > 0 or alpha < 1/255).  Both phases of the blending loops go
// through this one function, so they take the same decision on the same bits.
__device__ __forceinline__ bool eval_alpha(const float4 q0, const float2 q1xy, const float2 pixf, float2& d, float& G,
                                           float& alpha)
{
    d = {q0.x - pixf.x, q0.y - pixf.y};
    const float power = -0.5f * (q0.z * d.x * d.x + q1xy.x * d.y * d.y) - q0.w * d.x * d.y;
    if (power > 0.0f) return false;
    G = exp(power);
    alpha = min(0.99f, q1xy.y * G);
    return !(alpha < 1.0f / 255.0f);
}

// Pixel mask of one Gaussian over a warp's 8x4 pixel block (bit y * 8 + x = lane of that pixel): alpha is evaluated
// only at the pixels inside the Gaussian's safe box, by ONE lane, so 32 Gaussians are tested at once and a small
// splat costs a handful of evaluations instead of 32.  Same eval_alpha as the pixel's own walk: same bits.
__device__ __forceinline__ uint32_t block_pixel_mask(const float4 q0, const float2 q1xy, const float ex, const float ey,
                                                     const float sx0, const float sy0)
{
    const int x0 = max(0, (int)ceilf(q0.x - ex - sx0)), x1 = min(7, (int)floorf(q0.x + ex - sx0));
    const int y0 = max(0, (int)ceilf(q0.y - ey - sy0)), y1 = min(3, (int)floorf(q0.y + ey - sy0));
    uint32_t pm = 0;
    for (int y = y0; y <= y1; y++)
        for (int x = x0; x <= x1; x++) {
            float2 d;
            float G, alpha;
            if (eval_alpha(q0, q1xy, make_float2(sx0 + (float)x, sy0 + (float)y), d, G, alpha)) pm |= 1u << (y * 8 + x);
        }
    return pm;
}

// 32 x 32 bit matrix held one row per lane -> one column per lane (five exchanges of off-diagonal blocks).  Turns
// "lane v holds the pixel mask of visit v" into "lane p holds the visit mask of pixel p" and back.
__device__ __forceinline__ uint32_t warp_transpose32(uint32_t a, const int lane)
{
#pragma unroll
    for (int s = 0; s < 5; s++) {
        const int j = 16 >> s;
        const uint32_t m0 = s == 0 ? 0x0000FFFFu : s == 1 ? 0x00FF00FFu : s == 2 ? 0x0F0F0F0Fu
                          : s == 3 ? 0x33333333u : 0x55555555u;
        const uint32_t other = __shfl_xor_sync(0xffffffffu, a, j);
        a = (lane & j) ? ((a & ~m0) | ((other >> j) & m0)) : ((a & m0) | ((other & m0) << j));
    }
    return a;
}

// How densely the scene's splats cover the 8x4 pixel blocks they touch, measured by the forward pass: [0] = sum
// over visits of the pixels that pass the alpha test, [1] = visits.  The backward pass picks its walk from it
// without the host ever reading it: where a visit reaches most of its block (large splats: close or high-resolution
// views), evaluating every pixel against every visit and reducing with the butterfly is cheaper than walking
// per-pixel lists; where a visit reaches a few pixels (aerial views of small splats) it is the other way round.
// Both kernels are launched; the one that is not wanted returns at once.  Measured on B200 (pixels per visit ->
// backward per-pixel walk / every-pixel walk): 5.0 (6M-Gaussian ring scene, 1600x1200) 1.50 / 1.66 ms; 10.4 (1M
// Gaussians, 1920x1080) 0.40 / 0.32 ms; the threshold sits between.
#ifndef CGX_DENSE_PIXELS_PER_VISIT
#define CGX_DENSE_PIXELS_PER_VISIT 6
#endif
#ifndef CGX_FWD_MIN_LIST_CHUNK
#define CGX_FWD_MIN_LIST_CHUNK 20
#endif
#ifndef CGX_DENSE_PIXELS_PER_VISIT_FWD
#define CGX_DENSE_PIXELS_PER_VISIT_FWD 7
#endif
constexpr int DENSITY_SLOTS = 32;     // CTAs add into slot (tile id mod 32): no single hot address
constexpr size_t DENSITY_BYTES = DENSITY_SLOTS * 2 * sizeof(unsigned long long);
__device__ __forceinline__ bool density_says_dense(const unsigned long long* density)
{
    unsigned long long pixels = 0, visits = 0;
#pragma unroll 4
    for (int k = 0; k < DENSITY_SLOTS; k++) {
        pixels += density[2 * k];
        visits += density[2 * k + 1];
    }
    return pixels > (unsigned long long)CGX_DENSE_PIXELS_PER_VISIT * visits;
}

// ------------------------------------------------------------------------------------------------ pack
__global__ void __launch_bounds__(256)
pack_records_kernel(int P, const int* __restrict__ radii, const float2* __restrict__ means2D,
                    const float4* __restrict__ conic_opacity, const float* __restrict__ rgb,
                    const float* __restrict__ all_map, int render_geo, Record* __restrict__ records,
                    int* __restrict__ out_observe)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 2 * DENSITY_SLOTS) reinterpret_cast<unsigned long long*>(records + P)[i] = 0ull;
    if (i >= P) return;
    if (out_observe) out_observe[i] = 0;
    // Gaussians without a radius never enter a tile list: their record is never read, so it is not written
    if (radii && radii[i] <= 0) return;
    const float2 xy = means2D[i];
    const float4 co = conic_opacity[i];
    const float r = rgb[3 * i], g = rgb[3 * i + 1], b = rgb[3 * i + 2];
    float m[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    if (render_geo) {
#pragma unroll
        for (int k = 0; k < 5; k++) m[k] = all_map[5 * i + k];
    }
    Record rec;
    rec.q0 = {xy.x, xy.y, co.x, co.y};
    rec.q1 = {co.z, co.w, r, g};
    rec.q2 = {b, m[0], m[1], m[2]};
    const float2 ext = cull_extent(co.x, co.y, co.z, co.w);
    rec.q3 = {m[3], m[4], ext.x, ext.y};
    records[i] = rec;
}

constexpr int RENDER_THREADS = CGX_BLOCK_SIZE;
constexpr int RENDER_WARPS = RENDER_THREADS / 32;

struct FwdSmem {
    RecSlot rec[2][CGX_BLOCK_SIZE];
    int id[2][CGX_BLOCK_SIZE];
    uint8_t hits[RENDER_WARPS][CGX_BLOCK_SIZE];
    uint64_t bar[2];
    int red[4][RENDER_WARPS];
};

// MODE 0: every pixel looks at every Gaussian of the batch (the reference's loop); MODE 1: per-warp culling, then
// every lane looks at every surviving Gaussian; MODE 2 (default): per-warp culling, then the two-phase walk.
// All three produce identical bits.
template <int MODE>
__global__ void __launch_bounds__(RENDER_THREADS, 4)
render_fwd_kernel(const uint2* __restrict__ ranges, const uint32_t* __restrict__ point_list, int W, int H,
                  const float focal_x, const float focal_y, const float cx, const float cy,
                  const Record* __restrict__ records, float* __restrict__ final_T, uint32_t* __restrict__ n_contrib,
                  uint32_t* __restrict__ n_contrib2loss, const uint8_t* __restrict__ compute_locally,
                  const float* __restrict__ bg_color, float* __restrict__ out_color, int* __restrict__ out_observe,
                  float* __restrict__ out_all_map, float* __restrict__ out_plane_depth, const bool render_geo,
                  int* __restrict__ n_render_t, int* __restrict__ n_consider_t, int* __restrict__ n_contrib_t,
                  unsigned long long* __restrict__ density)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw);

    const uint32_t horizontal_blocks = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X;
    const uint32_t block_id = blockIdx.y * horizontal_blocks + blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    // warp w owns the 8x4 pixel block (w & 1, w >> 1) of the tile: compact footprints keep a small splat
    // inside few warps, which is what the per-warp culling (and the backward's per-warp reduction) pays for
    const uint32_t lx = (warp & 1) * 8 + (lane & 7), ly = (warp >> 1) * 4 + (lane >> 3);

    uint2 pix_min = {blockIdx.x * CGX_BLOCK_X, blockIdx.y * CGX_BLOCK_Y};
    uint2 pix = {pix_min.x + lx, pix_min.y + ly};
    uint32_t pix_id = W * pix.y + pix.x;
    float2 pixf = {(float)pix.x, (float)pix.y};
    const float2 ray = {(pixf.x - cx) / focal_x, (pixf.y - cy) / focal_y};
    bool inside = pix.x < W && pix.y < H;
    const size_t HW = (size_t)H * W;

    if (!compute_locally[block_id]) {
        // tiles owned by another rank: defined zeros in every image output
        if (inside) {
            final_T[pix_id] = 0.f;
            n_contrib[pix_id] = 0;
            n_contrib2loss[pix_id] = 0;
            for (int ch = 0; ch < CGX_NCH; ch++) out_color[ch * HW + pix_id] = 0.f;
            for (int ch = 0; ch < CGX_NMAP; ch++) out_all_map[ch * HW + pix_id] = 0.f;
            out_plane_depth[pix_id] = 0.f;
        }
        if (tid == 0) {
            const uint2 rg = ranges[block_id];
            n_render_t[block_id] = rg.y - rg.x;
            n_consider_t[block_id] = 0;
            n_contrib_t[block_id] = 0;
        }
        return;
    }

    bool done = !inside;
    uint2 range = ranges[block_id];
    const int rounds = ((range.y - range.x + CGX_BLOCK_SIZE - 1) / CGX_BLOCK_SIZE);
    int toDo = range.y - range.x;

    if (tid == 0) {
        mbar_init(&sm.bar[0], 1);
        mbar_init(&sm.bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // pixel block of this warp: columns [sx0, sx1], rows [sy0, sy1]
    const float sx0 = (float)(pix_min.x + (warp & 1) * 8), sx1 = sx0 + 7.f;
    const float sy0 = (float)(pix_min.y + (warp >> 1) * 4), sy1 = sy0 + 3.f;

    auto issue = [&](int batch, int buf) {
        const int progress = batch * CGX_BLOCK_SIZE + tid;
        const int n_valid = min(CGX_BLOCK_SIZE, (int)(range.y - range.x) - batch * CGX_BLOCK_SIZE);
        if (tid == 0) mbar_expect_tx(&sm.bar[buf], (uint32_t)n_valid * 64u);
        if (range.x + progress < range.y) {
            const int coll_id = point_list[range.x + progress];
            sm.id[buf][tid] = coll_id;
            bulk_load_64(&sm.rec[buf][tid], records + coll_id, &sm.bar[buf]);
        }
    };

    float T = 1.0f;
    uint32_t last_contributor = 0;
    uint32_t thread_n_contrib2loss = 0;
    float C[CGX_NCH] = {0};
    float All_map[CGX_NMAP] = {0};
    bool failed = false;
    uint32_t dens_rows = 0, dens_visits = 0;   // this warp's measured chunks: pixels reached, visits (warp-uniform)
    bool warp_dense = false;
    uint32_t chunk_no = 0;
    uint32_t lane_rows = 0;                    // pixels this lane blended in chunks that were not measured

    if (rounds > 0) issue(0, 0);

    for (int i = 0; i < rounds; i++, toDo -= CGX_BLOCK_SIZE) {
        const int buf = i & 1;
        if (!failed && !mbar_wait(&sm.bar[buf], (i >> 1) & 1)) failed = true;
        // End if the entire block votes that it is done rasterizing (also orders buffer reuse).
        int num_done = __syncthreads_count(done || failed);
        if (num_done == CGX_BLOCK_SIZE) break;
        if (i + 1 < rounds) issue(i + 1, buf ^ 1);

        const int nb = min(CGX_BLOCK_SIZE, toDo);
        const RecSlot* rec = sm.rec[buf];
        const int* ids = sm.id[buf];
        const uint32_t contributor_base = (uint32_t)i * CGX_BLOCK_SIZE;

        if (MODE >= 1) {
            // every warp compacts the Gaussians whose safe box meets its strip (order preserved)
            uint8_t* my_hits = sm.hits[warp];
            int n_hits = 0;
            for (int j0 = 0; j0 < nb; j0 += 32) {
                const int j = j0 + lane;
                bool hit = false;
                if (j < nb) {
                    const float4 q0 = rec[j].q0;
                    const float4 q3 = rec[j].q3;
                    hit = (q0.x + q3.z >= sx0) && (q0.x - q3.z <= sx1) && (q0.y + q3.w >= sy0) && (q0.y - q3.w <= sy1);
                }
                const uint32_t m = __ballot_sync(0xffffffffu, hit);
                if (hit) my_hits[n_hits + __popc(m & ((1u << lane) - 1u))] = (uint8_t)j;
                n_hits += __popc(m);
            }
            __syncwarp();
            if (MODE == 2) {
                for (int base = 0; base < n_hits; base += 32) {
                    if (__all_sync(0xffffffffu, done)) break;
                    const int g = min(32, n_hits - base);
                    // This warp's choice of walk follows the density of its own block so far (pixels reached per
                    // visit).  While it walks densely it measures one chunk in four.
                    // A short chunk gives per-pixel lists nothing to skip: it is walked by every pixel as well.
                    const bool short_chunk = g < CGX_FWD_MIN_LIST_CHUNK;
                    const bool measure = !short_chunk && (!warp_dense || (chunk_no++ & 3) == 0);
                    // phase 1: lane v tests Gaussian v against the block's pixels (only those in its safe box) ...
                    uint32_t pm = 0;
                    if (measure && lane < g && !(CGX_EXPERIMENT & 1)) {
                        const int j = my_hits[base + lane];
                        const float4 q3 = rec[j].q3;
                        pm = block_pixel_mask(rec[j].q0, *reinterpret_cast<const float2*>(&rec[j].q1), q3.z, q3.w, sx0,
                                              sy0);
                    }
                    if (measure) {
                        dens_rows += __reduce_add_sync(0xffffffffu, __popc(pm));
                        dens_visits += g;
                        warp_dense = dens_rows > (unsigned)CGX_DENSE_PIXELS_PER_VISIT_FWD * dens_visits;
                    }
                    const bool use_dense = warp_dense || short_chunk;
                    if (use_dense && !measure) dens_visits += g;      // its pixels are counted as they are blended
                    if (use_dense) {
                        // splats that cover most of the block: every pixel looks at every visit (no lists to build)
                        for (int v = 0; v < g; v++) {
                            if (done) continue;
                            const int j = my_hits[base + v];
                            const float4 q0 = rec[j].q0;
                            const float4 q1 = rec[j].q1;
                            float2 d;
                            float G, alpha;
                            if (!eval_alpha(q0, make_float2(q1.x, q1.y), pixf, d, G, alpha)) continue;
                            float test_T = T * (1 - alpha);
                            if (test_T < 0.0001f) {
                                done = true;
                                continue;
                            }
                            thread_n_contrib2loss++;
                            if (!measure) lane_rows++;
                            const float4 q2 = rec[j].q2;
                            const float feat[CGX_NCH] = {q1.z, q1.w, q2.x};
                            for (int ch = 0; ch < CGX_NCH; ch++) C[ch] += feat[ch] * alpha * T;
                            if (render_geo) {
                                const float4 q3 = rec[j].q3;
                                const float am[CGX_NMAP] = {q2.y, q2.z, q2.w, q3.x, q3.y};
                                for (int ch = 0; ch < CGX_NMAP; ch++) All_map[ch] += am[ch] * alpha * T;
                            }
                            if (T > 0.5) atomicAdd(&(out_observe[ids[j]]), 1);
                            T = test_T;
                            last_contributor = contributor_base + j + 1;
                        }
                        continue;
                    }
                    // ... and every pixel collects its own bit of each mask: one bit per visit that reaches it
                    uint32_t mine = warp_transpose32(pm, lane);      // pm is zero in the lanes beyond the chunk
                    if (done || (CGX_EXPERIMENT & 2)) mine = 0;
                    // phase 2: this pixel's own contributors, front to back
                    uint32_t seen_clear = 0;      // visits this pixel blended while its transmittance was above 0.5
                    while (mine) {
                        const int v = __ffs(mine) - 1;
                        mine &= mine - 1;
                        const int j = my_hits[base + v];
                        const float4 q0 = rec[j].q0;
                        const float4 q1 = rec[j].q1;
                        float2 d;
                        float G, alpha;
                        if (!eval_alpha(q0, make_float2(q1.x, q1.y), pixf, d, G, alpha)) continue;
                        float test_T = T * (1 - alpha);
                        if (test_T < 0.0001f) {
                            done = true;
                            break;
                        }
                        thread_n_contrib2loss++;
                        const float4 q2 = rec[j].q2;
                        const float feat[CGX_NCH] = {q1.z, q1.w, q2.x};
                        for (int ch = 0; ch < CGX_NCH; ch++) C[ch] += feat[ch] * alpha * T;
                        if (render_geo) {
                            const float4 q3 = rec[j].q3;
                            const float am[CGX_NMAP] = {q2.y, q2.z, q2.w, q3.x, q3.y};
                            for (int ch = 0; ch < CGX_NMAP; ch++) All_map[ch] += am[ch] * alpha * T;
                        }
                        if (T > 0.5) seen_clear |= 1u << v;
                        T = test_T;
                        last_contributor = contributor_base + j + 1;
                    }
                    // out_observe: one atomic per Gaussian with the number of such pixels (lanes walking their own
                    // lists would otherwise issue one atomic per pixel, to as many addresses as lanes)
                    if (__any_sync(0xffffffffu, seen_clear != 0)) {
                        const int cnt = __popc(warp_transpose32(seen_clear, lane));   // lane v: pixels of visit v
                        if (cnt) atomicAdd(&(out_observe[ids[my_hits[base + lane]]]), cnt);
                    }
                }
            } else
            for (int k = 0; !done && k < n_hits; k++) {
                const int j = my_hits[k];
                const float4 q0 = rec[j].q0;
                const float4 q1 = rec[j].q1;
                float2 xy = {q0.x, q0.y};
                float2 d = {xy.x - pixf.x, xy.y - pixf.y};
                float4 con_o = {q0.z, q0.w, q1.x, q1.y};
                float power = -0.5f * (con_o.x * d.x * d.x + con_o.z * d.y * d.y) - con_o.y * d.x * d.y;
                if (power > 0.0f) continue;
                float alpha = min(0.99f, con_o.w * exp(power));
                if (alpha < 1.0f / 255.0f) continue;
                float test_T = T * (1 - alpha);
                if (test_T < 0.0001f) {
                    done = true;
                    continue;
                }
                thread_n_contrib2loss++;
                const float4 q2 = rec[j].q2;
                const float feat[CGX_NCH] = {q1.z, q1.w, q2.x};
                for (int ch = 0; ch < CGX_NCH; ch++) C[ch] += feat[ch] * alpha * T;
                if (render_geo) {
                    const float4 q3 = rec[j].q3;
                    const float am[CGX_NMAP] = {q2.y, q2.z, q2.w, q3.x, q3.y};
                    for (int ch = 0; ch < CGX_NMAP; ch++) All_map[ch] += am[ch] * alpha * T;
                }
                if (T > 0.5) atomicAdd(&(out_observe[ids[j]]), 1);
                T = test_T;
                last_contributor = contributor_base + j + 1;
            }
        } else {
            for (int j = 0; !done && j < nb; j++) {
                const float4 q0 = rec[j].q0;
                const float4 q1 = rec[j].q1;
                float2 xy = {q0.x, q0.y};
                float2 d = {xy.x - pixf.x, xy.y - pixf.y};
                float4 con_o = {q0.z, q0.w, q1.x, q1.y};
                float power = -0.5f * (con_o.x * d.x * d.x + con_o.z * d.y * d.y) - con_o.y * d.x * d.y;
                if (power > 0.0f) continue;
                float alpha = min(0.99f, con_o.w * exp(power));
                if (alpha < 1.0f / 255.0f) continue;
                float test_T = T * (1 - alpha);
                if (test_T < 0.0001f) {
                    done = true;
                    continue;
                }
                thread_n_contrib2loss++;
                const float4 q2 = rec[j].q2;
                const float feat[CGX_NCH] = {q1.z, q1.w, q2.x};
                for (int ch = 0; ch < CGX_NCH; ch++) C[ch] += feat[ch] * alpha * T;
                if (render_geo) {
                    const float4 q3 = rec[j].q3;
                    const float am[CGX_NMAP] = {q2.y, q2.z, q2.w, q3.x, q3.y};
                    for (int ch = 0; ch < CGX_NMAP; ch++) All_map[ch] += am[ch] * alpha * T;
                }
                if (T > 0.5) atomicAdd(&(out_observe[ids[j]]), 1);
                T = test_T;
                last_contributor = contributor_base + j + 1;
            }
        }
    }
    if (failed && lane == 0) atomicExch(&g_status, CGX_ETIMEDOUT);

    if (inside) {
        final_T[pix_id] = T;
        n_contrib[pix_id] = last_contributor;
        n_contrib2loss[pix_id] = thread_n_contrib2loss;
        for (int ch = 0; ch < CGX_NCH; ch++) out_color[ch * HW + pix_id] = C[ch] + T * bg_color[ch];
        if (render_geo) {
            for (int ch = 0; ch < CGX_NMAP; ch++) out_all_map[ch * HW + pix_id] = All_map[ch];
            out_plane_depth[pix_id] = All_map[4] / -(All_map[0] * ray.x + All_map[1] * ray.y + All_map[2] + 1.0e-8);
        } else {
            for (int ch = 0; ch < CGX_NMAP; ch++) out_all_map[ch * HW + pix_id] = 0.f;
            out_plane_depth[pix_id] = 0.f;
        }
    }

    // per-tile sums of the two per-pixel counters (pixels outside the image count as 0)
    int a = inside ? (int)last_contributor : 0;
    int b = inside ? (int)thread_n_contrib2loss : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    dens_rows += __reduce_add_sync(0xffffffffu, lane_rows);
    if (lane == 0) {
        sm.red[0][warp] = a;
        sm.red[1][warp] = b;
        sm.red[2][warp] = (int)dens_rows;      // lane 0 adds the unmeasured chunks' pixels below
        sm.red[3][warp] = (int)dens_visits;
    }
    __syncthreads();
    if (tid == 0) {
        int sa = 0, sb = 0;
        unsigned long long dr = 0, dv = 0;
        for (int w = 0; w < RENDER_WARPS; w++) {
            sa += sm.red[0][w];
            sb += sm.red[1][w];
            dr += (unsigned)sm.red[2][w];
            dv += (unsigned)sm.red[3][w];
        }
        n_render_t[block_id] = range.y - range.x;
        n_consider_t[block_id] = sa;
        n_contrib_t[block_id] = sb;
        if (MODE == 2 && density && dv) {
            unsigned long long* slot = density + 2 * (block_id % DENSITY_SLOTS);
            atomicAdd(slot, dr);
            atomicAdd(slot + 1, dv);
        }
    }
}

__global__ void __launch_bounds__(RENDER_THREADS)
tile_stats_kernel(int W, int H, const uint2* __restrict__ ranges, const uint32_t* __restrict__ n_contrib_px,
                  const uint32_t* __restrict__ n_c2l_px, const uint8_t* __restrict__ compute_locally,
                  int* __restrict__ n_render, int* __restrict__ n_consider, int* __restrict__ n_contrib)
{
    __shared__ int red[2][RENDER_WARPS];
    const uint32_t block_id = blockIdx.y * gridDim.x + blockIdx.x;
    const int tid = threadIdx.y * CGX_BLOCK_X + threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const bool local = compute_locally[block_id];
    const uint32_t px = blockIdx.x * CGX_BLOCK_X + threadIdx.x, py = blockIdx.y * CGX_BLOCK_Y + threadIdx.y;
    const bool inside = px < (uint32_t)W && py < (uint32_t)H;
    int a = (local && inside) ? (int)n_contrib_px[(size_t)W * py + px] : 0;
    int b = (local && inside) ? (int)n_c2l_px[(size_t)W * py + px] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    if (lane == 0) {
        red[0][warp] = a;
        red[1][warp] = b;
    }
    __syncthreads();
    if (tid == 0) {
        int sa = 0, sb = 0;
        for (int w = 0; w < RENDER_WARPS; w++) {
            sa += red[0][w];
            sb += red[1][w];
        }
        const uint2 rg = ranges[block_id];
        n_render[block_id] = rg.y - rg.x;
        n_consider[block_id] = sa;
        n_contrib[block_id] = sb;
    }
}

// ------------------------------------------------------------------------------------------------ backward
#ifndef CGX_BWD_BATCH
#define CGX_BWD_BATCH 256
#endif
constexpr int BWD_BATCH = CGX_BWD_BATCH;   // records the backward kernels stage per round (per buffer)
static_assert(BWD_BATCH % 32 == 0 && BWD_BATCH <= RENDER_THREADS && BWD_BATCH <= 256, "one thread stages one record");

struct BwdOut {
    float* ptr[16];   // destination array of gradient term k
    int stride[16];   // floats per Gaussian in that array
};

struct BwdSmem {
    Record rec[2][BWD_BATCH];
    int id[2][BWD_BATCH];
    uint8_t hits[RENDER_WARPS][BWD_BATCH];
    uint64_t bar[2];
};

// Sum v[0..15] over the 32 lanes.  After the call, lane L holds in the return value the total of term
// term_of_lane(L) = 8*bit4 + 4*bit3 + 2*bit2 + bit1 of L (lanes 2m and 2m+1 hold the same total).
__device__ __forceinline__ float warp_reduce16(float (&v)[16], int lane)
{
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
    float w8[8];
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const float keep = b4 ? v[8 + k] : v[k];
        const float send = b4 ? v[k] : v[8 + k];
        w8[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
    float w4[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float keep = b3 ? w8[4 + k] : w8[k];
        const float send = b3 ? w8[k] : w8[4 + k];
        w4[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    float w2[2];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const float keep = b2 ? w4[2 + k] : w4[k];
        const float send = b2 ? w4[k] : w4[2 + k];
        w2[k] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    const float keep = b1 ? w2[1] : w2[0];
    const float send = b1 ? w2[0] : w2[1];
    float w1 = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
    return w1;
}

#ifndef CGX_BWD_MIN_CTAS
#define CGX_BWD_MIN_CTAS 3
#endif

// Per-pixel state of the backward walk (cuda_rasterizer/backward.cu:408-443): everything one pixel carries from
// one contributor to the next, back to front.
struct BwdPixel {
    float2 pixf;
    float T, T_final, last_alpha, bg_dot_dpixel;
    float dL_dpixel[CGX_NCH], dL_dout_all_map[CGX_NMAP];
    float accum_rec[CGX_NCH], last_color[CGX_NCH];
    float accum_all_map[CGX_NMAP], last_all_map[CGX_NMAP];
};

// One contribution (cuda_rasterizer/backward.cu:476-563 in the reference's operation order): advances the pixel's
// recurrences and writes the 16 gradient terms of (this pixel, this Gaussian) to v[]:
//   0,1 dL/dmean2D   2,3 |dL/dmean2D|   4,5,6 dL/dconic (xx, xy, yy)   7 dL/dopacity   8-10 dL/drgb   11-15 dL/dall_map
__device__ __forceinline__ void bwd_contribution(BwdPixel& px, const Record& r, const float2 d, const float G,
                                                 const float alpha, const bool render_geo, const float ddelx_dx,
                                                 const float ddely_dy, float (&v)[16])
{
    const float4 q0 = r.q0, q1 = r.q1, q2 = r.q2;
    // gradients carry a 1e-3 tolerance: one correctly rounded reciprocal serves both quotients
    const float inv_1ma = __frcp_rn(1.f - alpha);
    px.T = px.T * inv_1ma;
    const float dchannel_dcolor = alpha * px.T;
    float dL_dalpha = 0.0f;
    const float col[CGX_NCH] = {q1.z, q1.w, q2.x};
#pragma unroll
    for (int ch = 0; ch < CGX_NCH; ch++) {
        const float c = col[ch];
        px.accum_rec[ch] = px.last_alpha * px.last_color[ch] + (1.f - px.last_alpha) * px.accum_rec[ch];
        px.last_color[ch] = c;
        dL_dalpha += (c - px.accum_rec[ch]) * px.dL_dpixel[ch];
        v[8 + ch] = dchannel_dcolor * px.dL_dpixel[ch];
    }
    if (render_geo) {
        const float4 q3 = r.q3;
        const float am[CGX_NMAP] = {q2.y, q2.z, q2.w, q3.x, q3.y};
#pragma unroll
        for (int ch = 0; ch < CGX_NMAP; ch++) {
            const float c = am[ch];
            px.accum_all_map[ch] = px.last_alpha * px.last_all_map[ch] + (1.f - px.last_alpha) * px.accum_all_map[ch];
            px.last_all_map[ch] = c;
            dL_dalpha += (c - px.accum_all_map[ch]) * px.dL_dout_all_map[ch];
            v[11 + ch] = dchannel_dcolor * px.dL_dout_all_map[ch];
        }
    } else {
#pragma unroll
        for (int ch = 0; ch < CGX_NMAP; ch++) v[11 + ch] = 0.f;
    }
    dL_dalpha *= px.T;
    px.last_alpha = alpha;
    dL_dalpha += (-px.T_final * inv_1ma) * px.bg_dot_dpixel;

    const float dL_dG = q1.y * dL_dalpha;
    const float gdx = G * d.x;
    const float gdy = G * d.y;
    const float dG_ddelx = -gdx * q0.z - gdy * q0.w;
    const float dG_ddely = -gdy * q1.x - gdx * q0.w;
    v[0] = dL_dG * dG_ddelx * ddelx_dx;
    v[1] = dL_dG * dG_ddely * ddely_dy;
    v[2] = fabs(dL_dG * dG_ddelx * ddelx_dx);
    v[3] = fabs(dL_dG * dG_ddely * ddely_dy);
    v[4] = -0.5f * gdx * d.x * dL_dG;
    v[5] = -0.5f * gdx * d.y * dL_dG;
    v[6] = -0.5f * gdy * d.y * dL_dG;
    v[7] = G * dL_dalpha;
}

// Loads the pixel's cotangents and folds the plane-depth cotangent into the plane-map channels
// (cuda_rasterizer/backward.cu:379-443).
__device__ __forceinline__ void bwd_pixel_init(BwdPixel& px, bool inside, uint32_t pix_id, size_t HW, float2 ray,
                                               const float* __restrict__ bg_color, const float* __restrict__ final_Ts,
                                               const float* __restrict__ all_map_pixels,
                                               const float* __restrict__ dL_dpixels,
                                               const float* __restrict__ dL_dout_all_maps,
                                               const float* __restrict__ dL_dout_plane_depths, bool render_geo)
{
    px.T_final = inside ? final_Ts[pix_id] : 0;
    px.T = px.T_final;
    px.last_alpha = 0.f;
#pragma unroll
    for (int i = 0; i < CGX_NCH; i++) px.dL_dpixel[i] = px.accum_rec[i] = px.last_color[i] = 0.f;
#pragma unroll
    for (int i = 0; i < CGX_NMAP; i++) px.dL_dout_all_map[i] = px.accum_all_map[i] = px.last_all_map[i] = 0.f;
    if (inside) {
        for (int i = 0; i < CGX_NCH; i++) px.dL_dpixel[i] = dL_dpixels[i * HW + pix_id];
        if (render_geo) {
            for (int i = 0; i < CGX_NMAP; i++) px.dL_dout_all_map[i] = dL_dout_all_maps[i * HW + pix_id];
            const float3 normal = {all_map_pixels[pix_id], all_map_pixels[HW + pix_id], all_map_pixels[2 * HW + pix_id]};
            const float distance = all_map_pixels[4 * HW + pix_id];
            const float tmp = (normal.x * ray.x + normal.y * ray.y + normal.z + 1.0e-8);
            px.dL_dout_all_map[CGX_NMAP - 1] += (-dL_dout_plane_depths[pix_id] / tmp);
            px.dL_dout_all_map[0] += dL_dout_plane_depths[pix_id] * (distance / (tmp * tmp) * ray.x);
            px.dL_dout_all_map[1] += dL_dout_plane_depths[pix_id] * (distance / (tmp * tmp) * ray.y);
            px.dL_dout_all_map[2] += dL_dout_plane_depths[pix_id] * (distance / (tmp * tmp));
        }
    }
    px.bg_dot_dpixel = 0;
    for (int i = 0; i < CGX_NCH; i++) px.bg_dot_dpixel += bg_color[i] * px.dL_dpixel[i];
}

// The common head of both backward kernels: tile / pixel coordinates and the staging pipeline.
#define CGX_BWD_PROLOGUE()                                                                                           \
    /* two walks are launched when the forward pass measured the density: only the suitable one works */            \
    if (density) {                                                                                                   \
        __shared__ int s_not_mine;                                                                                   \
        if (threadIdx.x == 0) s_not_mine = density_says_dense(density) != (want_dense != 0);                         \
        __syncthreads();                                                                                             \
        if (s_not_mine) return;                                                                                      \
    }                                                                                                                \
    const uint32_t horizontal_blocks = (W + CGX_BLOCK_X - 1) / CGX_BLOCK_X;                                          \
    const uint32_t block_id = blockIdx.y * horizontal_blocks + blockIdx.x;                                           \
    if (!compute_locally[block_id]) return;                                                                          \
    const int tid = threadIdx.x;                                                                                     \
    const int lane = tid & 31, warp = tid >> 5;                                                                      \
    const uint32_t lx = (warp & 1) * 8 + (lane & 7), ly = (warp >> 1) * 4 + (lane >> 3); /* 8x4 block per warp */    \
    const uint2 pix_min = {blockIdx.x * CGX_BLOCK_X, blockIdx.y * CGX_BLOCK_Y};                                      \
    const uint2 pix = {pix_min.x + lx, pix_min.y + ly};                                                              \
    const uint32_t pix_id = W * pix.y + pix.x;                                                                       \
    const float2 pixf = {(float)pix.x, (float)pix.y};                                                                \
    /* double arithmetic (W * 0.5 is a double expression), narrowed to float afterwards */                           \
    const float2 ray = {(float)((pixf.x - W * 0.5) / fx), (float)((pixf.y - H * 0.5) / fy)};                         \
    const bool inside = pix.x < W && pix.y < H;                                                                      \
    const uint2 range = ranges[block_id];                                                                            \
    const size_t HW = (size_t)H * W;                                                                                 \
    const int rounds = ((range.y - range.x + BWD_BATCH - 1) / BWD_BATCH);                                  \
    int toDo = range.y - range.x;                                                                                    \
    if (tid == 0) {                                                                                                  \
        mbar_init(&sm.bar[0], 1);                                                                                    \
        mbar_init(&sm.bar[1], 1);                                                                                    \
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");                                           \
    }                                                                                                                \
    __syncthreads();                                                                                                 \
    const float sx0 = (float)(pix_min.x + (warp & 1) * 8), sx1 = sx0 + 7.f;                                          \
    const float sy0 = (float)(pix_min.y + (warp >> 1) * 4), sy1 = sy0 + 3.f;                                         \
    auto issue = [&](int batch, int buf) {                                                                           \
        const int progress = batch * BWD_BATCH + tid;                                                           \
        const int n_valid = min(BWD_BATCH, (int)(range.y - range.x) - batch * BWD_BATCH);                  \
        if (tid == 0) mbar_expect_tx(&sm.bar[buf], (uint32_t)n_valid * 64u);                                         \
        if (tid < BWD_BATCH && range.x + progress < range.y) {                                                       \
            const int coll_id = point_list[range.y - progress - 1]; /* back to front */                              \
            sm.id[buf][tid] = coll_id;                                                                               \
            bulk_load_64(&sm.rec[buf][tid], records + coll_id, &sm.bar[buf]);                                        \
        }                                                                                                            \
    };                                                                                                               \
    const uint32_t total = range.y - range.x;                                                                        \
    /* pixels outside the image take part in the votes only: nothing is ever "before their last contributor" */     \
    const int last_contributor = inside ? n_contrib[pix_id] : 0;                                                     \
    BwdPixel px;                                                                                                     \
    px.pixf = pixf;                                                                                                  \
    bwd_pixel_init(px, inside, pix_id, HW, ray, bg_color, final_Ts, all_map_pixels, dL_dpixels, dL_dout_all_maps,    \
                   dL_dout_plane_depths, render_geo);                                                                \
    const float ddelx_dx = 0.5 * W;                                                                                  \
    const float ddely_dy = 0.5 * H;                                                                                  \
    bool failed = false;                                                                                             \
    if (rounds > 0) issue(0, 0)

// Culls the staged batch against this warp's 8x4 pixel block: slots whose safe box meets the block, in order.
template <typename REC>
__device__ __forceinline__ int cull_batch(const REC* rec, int nb, int lane, float sx0, float sx1, float sy0,
                                          float sy1, uint8_t* my_hits)
{
    int n_hits = 0;
    for (int j0 = 0; j0 < nb; j0 += 32) {
        const int j = j0 + lane;
        bool hit = false;
        if (j < nb) {
            const float4 q0 = rec[j].q0;
            const float4 q3 = rec[j].q3;
            hit = (q0.x + q3.z >= sx0) && (q0.x - q3.z <= sx1) && (q0.y + q3.w >= sy0) && (q0.y - q3.w <= sy1);
        }
        const uint32_t m = __ballot_sync(0xffffffffu, hit);
        if (hit) my_hits[n_hits + __popc(m & ((1u << lane) - 1u))] = (uint8_t)j;
        n_hits += __popc(m);
    }
    __syncwarp();
    return n_hits;
}

// Reference-shaped walk: every lane looks at every (surviving) Gaussian; the 16 terms are reduced over the warp
// with the transposing butterfly.  Kept as the A/B partner of the two-phase kernel below.
template <bool CULL>
__global__ void __launch_bounds__(RENDER_THREADS, CGX_BWD_MIN_CTAS)
render_bwd_kernel(const uint2* __restrict__ ranges, const uint32_t* __restrict__ point_list, int W, int H, float fx,
                  float fy, const float* __restrict__ bg_color, const Record* __restrict__ records,
                  const float* __restrict__ all_map_pixels, const float* __restrict__ final_Ts,
                  const uint32_t* __restrict__ n_contrib, const uint8_t* __restrict__ compute_locally,
                  const float* __restrict__ dL_dpixels, const float* __restrict__ dL_dout_all_maps,
                  const float* __restrict__ dL_dout_plane_depths, const bool render_geo, BwdOut out,
                  const unsigned long long* __restrict__ density, int want_dense)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    BwdSmem& sm = *reinterpret_cast<BwdSmem*>(smem_raw);
    CGX_BWD_PROLOGUE();

    // destination of the term this lane owns after the butterfly
    const int my_term = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
    float* my_ptr = out.ptr[my_term];
    const int my_stride = out.stride[my_term];
    const bool my_write = (lane & 1) == 0 && my_ptr != nullptr;

    for (int i = 0; i < rounds; i++, toDo -= BWD_BATCH) {
        const int buf = i & 1;
        if (!mbar_wait(&sm.bar[buf], (i >> 1) & 1)) failed = true;
        const int any_failed = __syncthreads_or(failed);
        if (any_failed) break;
        if (i + 1 < rounds) issue(i + 1, buf ^ 1);

        const int nb = min(BWD_BATCH, toDo);
        const Record* rec = sm.rec[buf];
        const int* ids = sm.id[buf];
        // batch slot j holds sorted position range.y - 1 - (i*256 + j); its 0-based index in the tile list is
        // total - 1 - (i*256 + j), which is the reference's `contributor` after its decrement.
        const uint32_t idx_base = total - 1 - (uint32_t)i * BWD_BATCH;
        uint8_t* my_hits = sm.hits[warp];
        const int n_hits = CULL ? cull_batch(rec, nb, lane, sx0, sx1, sy0, sy1, my_hits) : nb;

        for (int k = 0; k < n_hits; k++) {
            const int j = CULL ? (int)my_hits[k] : k;
            const uint32_t contributor = idx_base - (uint32_t)j;
            float v[16];
            bool valid = false;
            if (contributor < (uint32_t)last_contributor) {
                float2 d;
                float G, alpha;
                if (eval_alpha(rec[j].q0, *reinterpret_cast<const float2*>(&rec[j].q1), pixf, d, G, alpha)) {
                    valid = true;
                    bwd_contribution(px, rec[j], d, G, alpha, render_geo, ddelx_dx, ddely_dy, v);
                }
            }
            const uint32_t vmask = __ballot_sync(0xffffffffu, valid);
            if (vmask == 0) continue;
            if (!valid) {
#pragma unroll
                for (int t = 0; t < 16; t++) v[t] = 0.f;
            }
            const float tot = warp_reduce16(v, lane);
            if (my_write) atomicAdd(my_ptr + (size_t)ids[j] * my_stride, tot);
        }
    }
    if (failed && lane == 0) atomicExch(&g_status, CGX_ETIMEDOUT);
}

// ---- two-phase backward
#ifndef CGX_BWD_CAP
#define CGX_BWD_CAP 60
#endif
constexpr int BWD_CAP = CGX_BWD_CAP;  // gradient rows a warp stages per group of visits (a visit adds at most 32);
                                      // 60 rows keep the CTA at 75 KB of shared memory: three CTAs per SM
constexpr int BWD_RS = 20;            // floats per staged row: 16 terms, 80-byte pitch (spreads rows over the banks)
static_assert(BWD_CAP >= 32 && BWD_CAP % 4 == 0, "a group must hold at least one full visit");

#ifndef CGX_BWD_REC80
#define CGX_BWD_REC80 0     // 1: 80-byte record pitch in the backward as well (needs a smaller gradient table)
#endif
#if CGX_BWD_REC80
typedef RecSlot BwdRec;
#else
typedef Record BwdRec;
#endif

struct BwdSmem2 {
    BwdRec rec[2][BWD_BATCH];
    int id[2][BWD_BATCH];
    float stage[RENDER_WARPS][BWD_CAP * BWD_RS];
    uint8_t hits[RENDER_WARPS][BWD_BATCH];
    uint64_t bar[2];
};

__global__ void __launch_bounds__(RENDER_THREADS, CGX_BWD_MIN_CTAS)
render_bwd2_kernel(const uint2* __restrict__ ranges, const uint32_t* __restrict__ point_list, int W, int H, float fx,
                   float fy, const float* __restrict__ bg_color, const Record* __restrict__ records,
                   const float* __restrict__ all_map_pixels, const float* __restrict__ final_Ts,
                   const uint32_t* __restrict__ n_contrib, const uint8_t* __restrict__ compute_locally,
                   const float* __restrict__ dL_dpixels, const float* __restrict__ dL_dout_all_maps,
                   const float* __restrict__ dL_dout_plane_depths, const bool render_geo, BwdOut out,
                   const unsigned long long* __restrict__ density, int want_dense)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    BwdSmem2& sm = *reinterpret_cast<BwdSmem2*>(smem_raw);
    CGX_BWD_PROLOGUE();

    // phase 3: four visits at a time, eight lanes each; lane t of a quarter owns gradient terms 2t and 2t + 1
    const int quarter = lane >> 3, term2 = (lane & 7) * 2;
    float* my_ptr0 = out.ptr[term2];
    float* my_ptr1 = out.ptr[term2 + 1];
    const int my_stride0 = out.stride[term2], my_stride1 = out.stride[term2 + 1];
    const uint32_t lanes_below = (1u << lane) - 1u;
    float* stage = sm.stage[warp];
    // a warp none of whose pixels has a contributor has nothing to do in any batch
    const bool warp_idle = __all_sync(0xffffffffu, last_contributor == 0);

    for (int i = 0; i < rounds; i++, toDo -= BWD_BATCH) {
        const int buf = i & 1;
        if (!mbar_wait(&sm.bar[buf], (i >> 1) & 1)) failed = true;
        const int any_failed = __syncthreads_or(failed);
        if (any_failed) break;
        if (i + 1 < rounds) issue(i + 1, buf ^ 1);
        if (warp_idle) continue;

        const int nb = min(BWD_BATCH, toDo);
        const BwdRec* rec = sm.rec[buf];
        const int* ids = sm.id[buf];
        // batch slot j holds sorted position range.y - 1 - (i*256 + j); its 0-based index in the tile list is
        // total - 1 - (i*256 + j), which is the reference's `contributor` after its decrement.
        const uint32_t idx_base = total - 1 - (uint32_t)i * BWD_BATCH;
        uint8_t* my_hits = sm.hits[warp];
        const int n_hits = cull_batch(rec, nb, lane, sx0, sx1, sy0, sy1, my_hits);

        for (int base = 0; base < n_hits; base += 32) {
            // ---- phase 1: which pixels does each visit reach?  Lane v keeps the pixel mask of visit v, every lane
            // keeps the visit mask of its own pixel.  A chunk of 32 visits is cut into groups whose rows fit the table.
            // Lane v tests Gaussian v against the block's pixels.
            const int g_max = min(32, n_hits - base);
            uint32_t pm = 0;
            if (lane < g_max && !(CGX_EXPERIMENT & 1)) {
                const int j = my_hits[base + lane];
                const float4 q3 = rec[j].q3;
                pm = block_pixel_mask(rec[j].q0, *reinterpret_cast<const float2*>(&rec[j].q1), q3.z, q3.w, sx0, sy0);
            }
            // Every pixel's bits of the chunk's masks at once (a bit-matrix transpose), cut down to the visits that lie
            // before the pixel's last contributor: the hits are in back-to-front order, so those are the visits from
            // some v_cut on, found by a search over the chunk's slots.  Transposed back, lane v holds the pixels
            // visit v really contributes to; a scan of their counts gives every visit its first table row.
            uint32_t mine_all = warp_transpose32(pm, lane);
            {
                const int thr = (int)idx_base - (int)last_contributor;   // valid: slot j > thr
                int lo = 0, hi = g_max;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if ((int)my_hits[base + mid] <= thr) lo = mid + 1;
                    else hi = mid;
                }
                mine_all = lo >= 32 ? 0u : (mine_all & (0xffffffffu << lo));
            }
            const uint32_t visit_mask = warp_transpose32(mine_all, lane);
            const int cnt = __popc(visit_mask);
            int cum = cnt;
#pragma unroll
            for (int dd = 1; dd < 32; dd <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, cum, dd);
                if (lane >= dd) cum += n;
            }
            int v0 = 0;      // visits [v0, v0 + g) of this chunk form the current group
            while (v0 < g_max) {
            // the group: as many visits from v0 on as the table holds (a visit alone always fits)
            const int before = v0 ? __shfl_sync(0xffffffffu, cum, v0 - 1) : 0;
            const int g = __popc(__ballot_sync(0xffffffffu, lane >= v0 && lane < g_max && cum - before <= BWD_CAP));
            const int rows = __shfl_sync(0xffffffffu, cum, v0 + g - 1) - before;
            uint32_t mine = (mine_all >> v0) & (g == 32 ? 0xffffffffu : ((1u << g) - 1u));
            if (rows) {
                const int first_row = cum - cnt - before;      // of visit `lane`, for the lanes of this group

                // ---- phase 2: every lane walks its own contributors, back to front, and stages their terms
                if (CGX_EXPERIMENT & 2) mine = 0;
                for (;;) {
                    const bool act = mine != 0;
                    if (!__any_sync(0xffffffffu, act)) break;
                    const int v = act ? __ffs(mine) - 1 : 0;
                    const uint32_t mv = __shfl_sync(0xffffffffu, visit_mask, v0 + v);
                    const int rv = __shfl_sync(0xffffffffu, first_row, v0 + v);
                    if (act) {
                        mine &= mine - 1;
                        const int j = my_hits[base + v0 + v];
                        float2 d;
                        float G, alpha;
                        eval_alpha(rec[j].q0, *reinterpret_cast<const float2*>(&rec[j].q1), pixf, d, G, alpha);
                        float val[16];
                        bwd_contribution(px, rec[j], d, G, alpha, render_geo, ddelx_dx, ddely_dy, val);
                        float4* row = reinterpret_cast<float4*>(stage + (rv + __popc(mv & lanes_below)) * BWD_RS);
                        row[0] = make_float4(val[0], val[1], val[2], val[3]);
                        row[1] = make_float4(val[4], val[5], val[6], val[7]);
                        row[2] = make_float4(val[8], val[9], val[10], val[11]);
                        row[3] = make_float4(val[12], val[13], val[14], val[15]);
                    }
                }
                __syncwarp();

                // ---- phase 3: four visits at a time, a quarter-warp each, lane = two terms: sum the visit's rows and
                // add the totals to the Gaussian's gradient with one atomic per term.  Visits without rows (no pixel
                // above the alpha threshold, or all of them behind their last contributor) are skipped: the quarters
                // take the next four visits that have some.
                uint32_t todo = __ballot_sync(0xffffffffu, lane >= v0 && lane < v0 + g && cnt > 0);
                if (CGX_EXPERIMENT & 4) todo = 0;
                while (todo) {
                    uint32_t t = todo;
                    if (quarter >= 1) t &= t - 1;
                    if (quarter >= 2) t &= t - 1;
                    if (quarter >= 3) t &= t - 1;
                    const int src = t ? __ffs(t) - 1 : 0;       // lane (= visit of the chunk) this quarter sums
                    const uint32_t mv = __shfl_sync(0xffffffffu, visit_mask, src);
                    const int rv = __shfl_sync(0xffffffffu, first_row, src);
                    if (t) {
                        const int n = __popc(mv);
                        const float2* p = reinterpret_cast<const float2*>(stage + rv * BWD_RS + term2);
                        float2 sum = p[0];
                        for (int r = 1; r < n; r++) {
                            const float2 x = p[r * (BWD_RS / 2)];
                            sum.x += x.x;
                            sum.y += x.y;
                        }
                        const size_t gid = (size_t)ids[my_hits[base + src]];
                        const bool go = !(CGX_EXPERIMENT & 8) || sum.x == 1.2345e-33f;
                        if (my_ptr0 && go) atomicAdd(my_ptr0 + gid * my_stride0, sum.x);
                        if (my_ptr1 && go) atomicAdd(my_ptr1 + gid * my_stride1, sum.y);
                    }
                    todo &= todo - 1;
                    todo &= todo - 1;
                    todo &= todo - 1;
                    todo &= todo - 1;
                }
                __syncwarp();
            }
            v0 += g;
            }
        }
    }
    if (failed && lane == 0) atomicExch(&g_status, CGX_ETIMEDOUT);
}

// Clears up to five float arrays in one launch (grid-stride over the concatenated index space).
struct ZeroJobs {
    float* ptr[5];
    long long n[5];
};
__global__ void __launch_bounds__(256) zero_arrays_kernel(ZeroJobs z)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
#pragma unroll
    for (int k = 0; k < 5; k++) {
        float* p = z.ptr[k];
        const long long n = z.n[k];
        if (!p) continue;
        if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
            float4* p4 = reinterpret_cast<float4*>(p);
            const long long n4 = n >> 2;
            for (long long i = t0; i < n4; i += stride) p4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (long long i = (n4 << 2) + t0; i < n; i += stride) p[i] = 0.f;
        } else {
            for (long long i = t0; i < n; i += stride) p[i] = 0.f;
        }
    }
}

}  // namespace cgx

using namespace cgx;

// P records, then the density counters the forward pass leaves for the backward pass
extern "C" int cgx_render_density_words(void) { return 2 * DENSITY_SLOTS; }
extern "C" int cgx_render_dense_threshold(void) { return CGX_DENSE_PIXELS_PER_VISIT; }

extern "C" size_t cgx_render_records_bytes(int P) { return (size_t)(P > 0 ? P : 0) * sizeof(Record) + DENSITY_BYTES; }

namespace cgx {
int fetch_render_status_async(int* out_pinned, cudaStream_t st)
{
    void* word = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&word, g_status);
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    return post_words(word, out_pinned, 1, st);
}
int fetch_render_status(int* out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, g_status, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    if (*out != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    }
    return CGX_OK;
}
}  // namespace cgx

// Test-only switch (cgx_raster_testing.h).  bit 0: per-warp culling; bit 1: always the reference-shaped walk (every
// lane looks at every surviving Gaussian, butterfly reduction in the backward); bit 2: always the two-phase walk.
// Default 1 = culling, walk chosen per launch from the density the forward pass measured (per chunk of visits in
// the forward itself).  All variants give the same forward bits and gradients equal to rounding.
static int g_render_variant = 1;

extern "C" int cgx_set_render_variant(int variant)
{
    g_render_variant = variant & 7;
    return CGX_OK;
}

extern "C" int cgx_render_fwd(int P, int W, int H, float tanfovx, float tanfovy, const uint32_t* ranges,
                              const uint32_t* point_list, const int32_t* radii, const float* means2D, const float* rgb, const float* all_map,
                              const float* conic_opacity, const uint8_t* compute_locally, const float* bg,
                              int render_geo, void* records, float* final_T, uint32_t* n_contrib,
                              uint32_t* n_contrib2loss, float* out_color, int32_t* out_observe, float* out_all_map,
                              float* out_plane_depth, int32_t* n_render_t, int32_t* n_consider_t, int32_t* n_contrib_t,
                              void* stream)
{
    if (P < 0 || W <= 0 || H <= 0) return CGX_EINVAL;
    if (!ranges || !compute_locally || !bg || !final_T || !n_contrib || !n_contrib2loss || !out_color ||
        !out_all_map || !out_plane_depth || !n_render_t || !n_consider_t || !n_contrib_t)
        return CGX_EINVAL;
    if (P > 0 && (!means2D || !rgb || !conic_opacity || !records || !out_observe || (render_geo && !all_map)))
        return CGX_EINVAL;
    if (P > 0 && (((uintptr_t)means2D & 7) || !aligned16(conic_opacity) || !aligned16(records))) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if (P > 0)
        pack_records_kernel<<<(P + 255) / 256, 256, 0, st>>>(P, radii, (const float2*)means2D,
                                                             (const float4*)conic_opacity, rgb, all_map, render_geo,
                                                             (Record*)records, out_observe);
    const float focal_y = H / (2.0f * tanfovy);
    const float focal_x = W / (2.0f * tanfovx);
    const dim3 grid((W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y, 1);
    const dim3 block(RENDER_THREADS, 1, 1);
    const size_t smem = sizeof(FwdSmem);
    cudaError_t e = cudaSuccess;
#define CGX_LAUNCH_FWD(MODE)                                                                                         \
    do {                                                                                                            \
        e = cudaFuncSetAttribute(render_fwd_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }                                              \
        render_fwd_kernel<MODE><<<grid, block, smem, st>>>(                                                         \
            (const uint2*)ranges, point_list, W, H, focal_x, focal_y, float(W * 0.5f), float(H * 0.5f),             \
            (const Record*)records, final_T, n_contrib, n_contrib2loss, compute_locally, bg, out_color, out_observe, \
            out_all_map, out_plane_depth, render_geo != 0, n_render_t, n_consider_t, n_contrib_t,                   \
            (MODE == 2 && P > 0) ? reinterpret_cast<unsigned long long*>((Record*)records + P) : nullptr);          \
    } while (0)
    if (!(g_render_variant & 1))
        CGX_LAUNCH_FWD(0);
    else if (g_render_variant & 2)
        CGX_LAUNCH_FWD(1);
    else
        CGX_LAUNCH_FWD(2);
#undef CGX_LAUNCH_FWD
    return check_launch(P > 0 ? 2 : 1);
}

extern "C" int cgx_tile_stats(int W, int H, const uint32_t* ranges, const uint32_t* n_contrib_px,
                              const uint32_t* n_contrib2loss_px, const uint8_t* compute_locally, int32_t* n_render,
                              int32_t* n_consider, int32_t* n_contrib, void* stream)
{
    if (W <= 0 || H <= 0 || !ranges || !n_contrib_px || !n_contrib2loss_px || !compute_locally || !n_render ||
        !n_consider || !n_contrib)
        return CGX_EINVAL;
    const dim3 grid((W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y, 1);
    const dim3 block(CGX_BLOCK_X, CGX_BLOCK_Y, 1);
    tile_stats_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(W, H, (const uint2*)ranges, n_contrib_px,
                                                               n_contrib2loss_px, compute_locally, n_render,
                                                               n_consider, n_contrib);
    return check_launch();
}

extern "C" int cgx_render_bwd(int P, int W, int H, float tanfovx, float tanfovy, const uint32_t* ranges,
                              const uint32_t* point_list, const float* bg, const void* records,
                              const float* all_map_pixels, const float* final_T, const uint32_t* n_contrib,
                              const uint8_t* compute_locally, const float* dL_dcolor, const float* dL_dout_all_map,
                              const float* dL_dout_plane_depth, int render_geo, float* dL_dmeans2D,
                              float* dL_dmeans2D_abs, float* dL_dconic_opacity, float* dL_drgb, float* dL_dall_map,
                              int walk, void* stream)
{
    if (P < 0 || W <= 0 || H <= 0 || walk < 0 || walk > 2) return CGX_EINVAL;
    if (P == 0) return CGX_OK;
    if (!ranges) return CGX_EINVAL;
    if (!bg || !records || !final_T || !n_contrib || !compute_locally || !dL_dcolor || !dL_dmeans2D ||
        !dL_dmeans2D_abs || !dL_dconic_opacity || !dL_drgb || !dL_dall_map)
        return CGX_EINVAL;
    if (render_geo && (!all_map_pixels || !dL_dout_all_map || !dL_dout_plane_depth)) return CGX_EINVAL;
    if (!aligned16(records)) return CGX_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
    {
        // the five gradient arrays start at zero: one launch clears all of them
        ZeroJobs z;
        float* arrs[5] = {dL_dmeans2D, dL_dmeans2D_abs, dL_dconic_opacity, dL_drgb, dL_dall_map};
        const int widths[5] = {2, 3, 4, 3, 5};
        for (int k = 0; k < 5; k++) {
            z.ptr[k] = arrs[k];
            z.n[k] = (long long)P * widths[k];
        }
        zero_arrays_kernel<<<148 * 8, 256, 0, st>>>(z);
    }

    BwdOut out;
    float* ptrs[16] = {dL_dmeans2D, dL_dmeans2D + 1, dL_dmeans2D_abs, dL_dmeans2D_abs + 1,
                       dL_dconic_opacity, dL_dconic_opacity + 1, dL_dconic_opacity + 2, dL_dconic_opacity + 3,
                       dL_drgb, dL_drgb + 1, dL_drgb + 2,
                       dL_dall_map, dL_dall_map + 1, dL_dall_map + 2, dL_dall_map + 3, dL_dall_map + 4};
    const int strides[16] = {2, 2, 3, 3, 4, 4, 4, 4, 3, 3, 3, 5, 5, 5, 5, 5};
    for (int k = 0; k < 16; k++) {
        out.ptr[k] = ptrs[k];
        out.stride[k] = strides[k];
    }
    if (!render_geo)
        for (int k = 11; k < 16; k++) out.ptr[k] = nullptr;

    const float focal_y = H / (2.0f * tanfovy);
    const float focal_x = W / (2.0f * tanfovx);
    const dim3 grid((W + CGX_BLOCK_X - 1) / CGX_BLOCK_X, (H + CGX_BLOCK_Y - 1) / CGX_BLOCK_Y, 1);
    const dim3 block(RENDER_THREADS, 1, 1);
    // default: the forward pass left the scene's density beside the records; both walks are queued and the one the
    // density does not call for returns at once (no host read).  Forced variants pass no density.
    const unsigned long long* density = reinterpret_cast<const unsigned long long*>((const Record*)records + P);
#define CGX_LAUNCH_BWD(KERNEL, SMEM, DENSITY, WANT_DENSE)                                                            \
    do {                                                                                                            \
        e = cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM));                 \
        if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }                                              \
        KERNEL<<<grid, block, (SMEM), st>>>(                                                                        \
            (const uint2*)ranges, point_list, W, H, focal_x, focal_y, bg, (const Record*)records, all_map_pixels,   \
            final_T, n_contrib, compute_locally, dL_dcolor, dL_dout_all_map, dL_dout_plane_depth, render_geo != 0,  \
            out, DENSITY, WANT_DENSE);                                                                              \
    } while (0)
    int launched = 2;
    if (!(g_render_variant & 1))
        CGX_LAUNCH_BWD(render_bwd_kernel<false>, sizeof(BwdSmem), nullptr, 0);
    else if (g_render_variant & 2)
        CGX_LAUNCH_BWD(render_bwd_kernel<true>, sizeof(BwdSmem), nullptr, 0);
    else if (g_render_variant & 4)
        CGX_LAUNCH_BWD(render_bwd2_kernel, sizeof(BwdSmem2), nullptr, 0);
    else if (walk == 1)
        CGX_LAUNCH_BWD(render_bwd2_kernel, sizeof(BwdSmem2), nullptr, 0);       // the caller has read the density
    else if (walk == 2)
        CGX_LAUNCH_BWD(render_bwd_kernel<true>, sizeof(BwdSmem), nullptr, 0);
    else {
        CGX_LAUNCH_BWD(render_bwd2_kernel, sizeof(BwdSmem2), density, 0);
        CGX_LAUNCH_BWD(render_bwd_kernel<true>, sizeof(BwdSmem), density, 1);
        launched = 3;
    }
#undef CGX_LAUNCH_BWD
    return check_launch(launched);
}
