/*
 * cgx_raster — C ABI of the B200 (sm_100a) Gaussian rasterizer hot path.
 *
 * Drop-in boundary for the CityGS-X `diff_gaussian_rasterization._C` extension
 * (reference project paths: RAST = submodule_cityx/diff-gaussian-rasterization).
 * Every entry point takes plain device pointers and sizes, launches on the
 * given CUDA stream (passed as void*, i.e. a cudaStream_t), returns an int
 * status (0 = ok) and never allocates, frees or retains memory: the caller
 * owns inputs, outputs and workspaces.  Unless stated otherwise all pointers
 * are DEVICE pointers, floats are fp32, matrices are 16 floats in the
 * reference's row-vector convention (translation in elements 12..14), and
 * per-Gaussian arrays are row-major AoS exactly as the reference's tensors.
 *
 * Calls are asynchronous with respect to the host unless the comment says
 * "host-synchronous".
 */
#ifndef CGX_RASTER_H
#define CGX_RASTER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define CGX_OK 0
#define CGX_EINVAL 22      /* bad shape / null pointer / misaligned pointer            */
#define CGX_ENOMEM 12      /* caller-provided workspace or capacity too small           */
#define CGX_ETIMEDOUT 110  /* a bounded device-side wait gave up                        */
#define CGX_ECUDA 5        /* CUDA runtime reported an error (see cgx_last_cuda_error)  */

const char* cgx_strerror(int status);
/* Text of the last CUDA runtime error seen by this library on this thread. */
const char* cgx_last_cuda_error(void);
/* Library version string. */
const char* cgx_version(void);
/* Number of kernels this library has launched in this process (all entry points, all streams). */
unsigned long long cgx_launch_count(void);

/* GetBlockXY (RAST/rasterize_points.cu:858-861): tile size and 1-D block size. */
int cgx_block_xy(int* block_x, int* block_y, int* one_dim_block);

/* getHigherMsb (RAST/cuda_rasterizer/rasterizer_impl.cu:39-54). */
uint32_t cgx_higher_msb(uint32_t n);

/* ------------------------------------------------------------------ per-Gaussian stages */

/* markVisible -> checkFrustum (RAST/rasterize_points.cu:39-58,
 * RAST/cuda_rasterizer/rasterizer_impl.cu:58-70,147-159): present[i] = view-space z > 0.
 * present: P bytes (bool). */
int cgx_mark_visible(int P, const float* means3D, const float* viewmatrix, uint8_t* present, void* stream);

/* PreprocessGaussiansCUDA -> preprocessForward -> preprocessCUDA
 * (RAST/rasterize_points.cu:63-143, RAST/cuda_rasterizer/rasterizer_impl.cu:336-425,
 * RAST/cuda_rasterizer/forward.cu:156-259).  Writes EVERY element of every output
 * (zeros where the reference leaves its zero-filled allocation untouched), so outputs
 * may be uninitialised memory.
 *   means3D (P,3) scales (P,3) rotations (P,4) [r,x,y,z, not normalised] opacities (P,1)
 *   -> means2D (P,2) depths (P) radii int32 (P) cov3D (P,6) conic_opacity (P,4)          */
int cgx_preprocess_fwd(int P, const float* means3D, const float* scales, float scale_modifier,
                       const float* rotations, const float* opacities, const float* viewmatrix,
                       const float* projmatrix, int W, int H, float tanfovx, float tanfovy,
                       float* means2D, float* depths, int32_t* radii, float* cov3D, float* conic_opacity,
                       void* stream);

/* RasterizeGaussiansfilterCUDA -> visible_filter -> filter_preprocessCUDA
 * (RAST/rasterize_points.cu:865-930, RAST/cuda_rasterizer/forward.cu:545-620): radii only. */
int cgx_filter_preprocess(int P, const float* means3D, const float* scales, float scale_modifier,
                          const float* rotations, const float* viewmatrix, const float* projmatrix,
                          int W, int H, float tanfovx, float tanfovy, int32_t* radii, void* stream);
/* The same filter for callers that hold precomputed 3-D covariances (six floats per Gaussian, upper triangle) instead
 * of scales and rotations: the `cov3D_precomp` branch of filter_preprocessCUDA
 * (RAST/cuda_rasterizer/forward.cu:585-595). */
int cgx_filter_preprocess_cov3d(int P, const float* means3D, const float* cov3D_precomp, const float* viewmatrix,
                                const float* projmatrix, int W, int H, float tanfovx, float tanfovy,
                                int32_t* radii, void* stream);

/* Optional SH stage, computeColorFromSH (RAST/cuda_rasterizer/forward.cu:21-72; compiled out of the
 * reference's kernel, kept here as a switchable stage).  sh (P,M,3), campos 3 floats (device),
 * -> rgb (P,3), clamped (P,3) bytes. */
int cgx_sh_to_rgb(int P, int degree, int M, const float* means3D, const float* campos, const float* sh,
                  float* rgb, uint8_t* clamped, void* stream);

/* PreprocessGaussiansBackwardCUDA -> preprocessBackward -> computeCov2DCUDA + preprocessCUDA(bwd)
 * (RAST/rasterize_points.cu:146-234, RAST/cuda_rasterizer/backward.cu:69-321,578-641), one fused
 * kernel, including the (P,4) -> (P,2,2)+(P,1) cotangent repack of rasterize_points.cu:181-194.
 *   dL_dmeans2D (P,2), dL_dconic_opacity (P,4)
 *   -> dL_dmeans3D (P,3) dL_dscales (P,3) dL_drotations (P,4) dL_dopacity (P,1); every element written. */
int cgx_preprocess_bwd(int P, const float* means3D, const float* scales, float scale_modifier,
                       const float* rotations, const int32_t* radii, const float* viewmatrix,
                       const float* projmatrix, int W, int H, float tanfovx, float tanfovy,
                       const float* dL_dmeans2D, const float* dL_dconic_opacity,
                       float* dL_dmeans3D, float* dL_dscales, float* dL_drotations, float* dL_dopacity,
                       void* stream);

/* The caller's per-camera loop around preprocess (gaussian_renderer/__init__.py:966-1023) as ONE launch over a
 * batch of B <= 16 cameras: parameters are read once and projected into every camera (outputs per camera, same
 * bits as cgx_preprocess_fwd; the camera-independent covariance is not written); the backward reads them once
 * and writes the gradients already summed over the cameras.  Pointer arrays are host arrays of device pointers. */
typedef struct cgx_camera {
    const float* viewmatrix;   /* device, 16 floats */
    const float* projmatrix;   /* device, 16 floats */
    float tanfovx, tanfovy;
    int W, H;
} cgx_camera;
int cgx_preprocess_fwd_batched(int P, int B, const float* means3D, const float* scales, float scale_modifier,
                               const float* rotations, const float* opacities, const cgx_camera* cams,
                               float* const* means2D, float* const* depths, int32_t* const* radii,
                               float* const* conic_opacity, void* stream);
int cgx_preprocess_bwd_batched(int P, int B, const float* means3D, const float* scales, float scale_modifier,
                               const float* rotations, const cgx_camera* cams, const int32_t* const* radii,
                               const float* const* dL_dmeans2D, const float* const* dL_dconic_opacity,
                               float* dL_dmeans3D, float* dL_dscales, float* dL_drotations, float* dL_dopacity,
                               void* stream);
/* The same two launches with the plane descriptors of cgx_all_map_fwd / cgx_all_map_bwd fused in: the forward
 * also writes all_map[b] (P,5) for camera b (zeros where the radius is 0), the backward also takes
 * dL_dall_map[b] (P,5) and adds its contribution to dL_dmeans3D and dL_drotations.  campos[b]: device pointer to
 * camera b's centre (3 floats).  all_map / dL_dall_map (and campos with them) may be null, or hold null entries
 * for cameras that need no descriptors. */
int cgx_preprocess_fwd_batched_planes(int P, int B, const float* means3D, const float* scales, float scale_modifier,
                                      const float* rotations, const float* opacities, const cgx_camera* cams,
                                      const float* const* campos, float* const* means2D, float* const* depths,
                                      int32_t* const* radii, float* const* conic_opacity, float* const* all_map,
                                      void* stream);
int cgx_preprocess_bwd_batched_planes(int P, int B, const float* means3D, const float* scales, float scale_modifier,
                                      const float* rotations, const cgx_camera* cams, const float* const* campos,
                                      const int32_t* const* radii, const float* const* dL_dmeans2D,
                                      const float* const* dL_dconic_opacity, const float* const* dL_dall_map,
                                      float* dL_dmeans3D, float* dL_dscales, float* dL_drotations,
                                      float* dL_dopacity, void* stream);

/* The owner's backward driven by the gradient rows that came back through the exchange, instead of by dense
 * per-camera cotangent arrays: rows[r] = ncols floats [dL/dmeans2D 2 | dL/drgb 3 (ignored) | dL/dconic_opacity 4 |
 * dL/dall_map 5 when ncols = 14], row_gaussian[r] = local index of the Gaussian the row belongs to, segments[] says
 * which rows belong to which camera (at most 64 segments per call, host array).  A Gaussian may own several rows of
 * one camera (it was sent to two ranks); Gaussians without rows get zero gradients.  Replaces, for the
 * peer-to-peer exchange, the scatter of returned rows into (P, .) arrays followed by preprocessBackward per camera
 * (autograd through the differentiable all_to_all of gaussian_renderer/__init__.py:660-676; cuda_rasterizer/backward.cu:203-321,80-198).
 * workspace: cgx_preprocess_bwd_rows_workspace_bytes(P) bytes, 16-byte aligned, cleared by the call.  Sums over rows
 * use atomics:
 * results agree with cgx_preprocess_bwd_batched_planes to float rounding, not bit for bit. */
typedef struct cgx_row_segment {
    long long start;   /* first row of the segment */
    long long count;   /* rows in the segment */
    int camera;        /* index into cams[] */
    int reserved;
} cgx_row_segment;
size_t cgx_preprocess_bwd_rows_workspace_bytes(int P);
int cgx_preprocess_bwd_rows(int P, int n_segments, const cgx_row_segment* segments, int ncols, const float* rows,
                            const int32_t* row_gaussian, const float* means3D, const float* scales,
                            float scale_modifier, const float* rotations, int B, const cgx_camera* cams,
                            const float* const* campos, void* workspace, size_t workspace_bytes, float* dL_dmeans3D,
                            float* dL_dscales, float* dL_drotations, float* dL_dopacity, void* stream);

/* PGSR per-Gaussian plane descriptor [normal_cam(3), 1, plane distance] for one camera: the
 * tensor code of the reference's caller (gaussian_renderer/__init__.py:1501-1518) as one kernel.
 * radii optional: rows with radius <= 0 get zeros.  all_map (P,5). */
int cgx_all_map_fwd(int P, const float* means3D, const float* scales, const float* rotations,
                    const int32_t* radii, const float* viewmatrix, const float* campos, float* all_map,
                    void* stream);
/* Its backward (the autograd graph of the same tensor code): cotangent of all_map (P,5) -> cotangents of means3D
 * (P,3) and of the raw quaternions (P,4), both WRITTEN; scales receive no gradient (they only select the column). */
int cgx_all_map_bwd(int P, const float* means3D, const float* scales, const float* rotations,
                    const int32_t* radii, const float* viewmatrix, const float* campos, const float* dL_dall_map,
                    float* dL_dmeans3D, float* dL_drotations, void* stream);

/* ------------------------------------------------------------------ strip loss */

/* Masked L1 and masked 11x11 Gaussian-window SSIM sums of a rendered strip against its ground truth, and the
 * gradient towards the rendered strip: pixelwise_l1_with_mask / pixelwise_ssim_with_mask (utils/loss_utils.py:88-132,
 * window from :27-43, zero padding as conv2d(padding=5)) and their autograd backward as two kernels.
 * img, gt: (C,H,W) float; mask: (H,W) bytes, 0 = excluded, optional.  sums: two DOUBLES, both written,
 * sums[0] = sum mask*|img-gt|, sums[1] = sum mask*SSIM (the per-CTA partial sums are accumulated in double, so
 * the result does not depend on their order).  d_mu / d_xx / d_xy: (C,H,W) each, written by the forward when given
 * (all three or none): the masked partial derivatives of the SSIM map with respect to the window moments E[x],
 * E[x^2], E[xy], which is all the backward needs.  weights: 2 floats ON THE DEVICE = dL/dsums[0], dL/dsums[1] (no
 * host read of the incoming gradient).  dL_dimg (C,H,W) is written. */
int cgx_strip_loss_fwd(int C, int H, int W, const float* img, const float* gt, const uint8_t* mask, double* sums,
                       float* d_mu, float* d_xx, float* d_xy, void* stream);
int cgx_strip_loss_bwd(int C, int H, int W, const float* img, const float* gt, const uint8_t* mask,
                       const float* weights, const float* d_mu, const float* d_xx, const float* d_xy, float* dL_dimg,
                       void* stream);

/* Normal image of a depth image and its backward: render_normal (gaussian_renderer/__init__.py:1311-1323) at
 * scale 1 without offsets, i.e. normal_from_depth_image / depth_pcd2normal (utils/graphics_utils.py:87-152):
 * camera-space points z * ((x - cx)/fx, (y - cy)/fy, 1), normalised cross product of the horizontal and vertical
 * central differences, zero on the one-pixel border.  depth (H,W) -> normal (3,H,W); dL_dnormal (3,H,W) ->
 * dL_ddepth (H,W), written. */
int cgx_depth_normal_fwd(int H, int W, float fx, float fy, float cx, float cy, const float* depth, float* normal,
                         void* stream);
int cgx_depth_normal_bwd(int H, int W, float fx, float fy, float cx, float cy, const float* depth,
                         const float* dL_dnormal, float* dL_ddepth, void* stream);

/* ------------------------------------------------------------------ distribution */

/* GetLocal2jIdsBoolCUDA -> getTouchedIdsBool (RAST/rasterize_points.cu:445-524).
 * tile_bounds: int32 (ws+1) linear tile ids (= division_pos * TILE_X). mask: (P, ws) bytes, every
 * element written. */
int cgx_local2j_mask(int P, int H, int W, int ws, const float* means2D, const int32_t* radii,
                     const int32_t* tile_bounds, int avoid_pixel_all2all, uint8_t* mask, void* stream);

/* Fused replacement of the caller loop around get_local2j_ids_bool (mask -> nonzero -> index-gather
 * -> concat; gaussian_renderer/workload_division.py:721-744, gaussian_renderer/__init__.py:612-666,
 * 709-716).  Two passes over one camera's local Gaussians:
 *   cgx_local2j_count : counts (ws) int32 (device) = rows whose tile span touches each destination's band.
 *   cgx_local2j_pack  : writes those rows, ascending local index per destination (the order nonzero()
 *                       yields), starting at row send_row_offset[j] (host array, ws entries) of
 *                       send_buffer (rows of 19 floats: means2D 2 | rgb 3 | conic_opacity 4 | means3D 3 |
 *                       scales 3 | rotations 4), send_aux (rows of 2 floats: radius as float | depth) and
 *                       send_index (int32 source row, optional).
 * workspace: cgx_local2j_workspace_bytes(P, ws) bytes, the SAME buffer for both calls of a camera. */
size_t cgx_local2j_workspace_bytes(int P, int ws);
int cgx_local2j_count(int P, int H, int W, int ws, const float* means2D, const int32_t* radii,
                      const int32_t* tile_bounds, int avoid_pixel_all2all, int32_t* counts,
                      void* workspace, size_t workspace_bytes, void* stream);
int cgx_local2j_pack(int P, int H, int W, int ws, const float* means2D, const float* rgb,
                     const float* conic_opacity, const float* means3D, const float* scales,
                     const float* rotations, const int32_t* radii, const float* depths,
                     const int32_t* tile_bounds, int avoid_pixel_all2all,
                     const int64_t* send_row_offset, float* send_buffer, float* send_aux, int32_t* send_index,
                     void* workspace, size_t workspace_bytes, void* stream);
/* Backward of the pack (the reference gets it from autograd through index/cat): the 19-float gradient rows
 * of the listed row ranges [range_start[r], range_stop[r]) (host arrays, n_ranges <= 32) are added onto the
 * per-source-row gradient arrays through send_index (a source row can appear under several destinations).
 * d_rgb, d_means3D, d_scales, d_rotations may be NULL. */
int cgx_unpack_grad_add(int n_ranges, const int64_t* range_start, const int64_t* range_stop,
                        const float* grad_rows, const int32_t* send_index,
                        float* d_means2D, float* d_rgb, float* d_conic_opacity, float* d_means3D,
                        float* d_scales, float* d_rotations, void* stream);

/* Receiver side of the exchange.  Rows arrive source-rank major; the rows of one camera are one segment per
 * source rank: segment r = rows [seg_start[r], seg_start[r] + seg_count[r]) of the receive buffers (host
 * arrays, n_segments <= 32).  cgx_unpack_rows concatenates a camera's segments (source rank ascending, as
 * gaussian_renderer/__init__.py:683-696 does with split + cat) into the contiguous per-camera tensors
 * means2D (n,2) rgb (n,3) conic_opacity (n,4) means3D (n,3) scales (n,3) rotations (n,4) radii int32 (n)
 * depths (n); cgx_pack_grad_rows is its backward: gradient tensors (any may be NULL = zero) back into
 * 19-float rows at the same places. */
int cgx_unpack_rows(int n_segments, const int64_t* seg_start, const int64_t* seg_count, const float* rows,
                    const float* aux, float* means2D, float* rgb, float* conic_opacity, float* means3D,
                    float* scales, float* rotations, int32_t* radii, float* depths, void* stream);
int cgx_pack_grad_rows(int n_segments, const int64_t* seg_start, const int64_t* seg_count,
                       const float* d_means2D, const float* d_rgb, const float* d_conic_opacity,
                       const float* d_means3D, const float* d_scales, const float* d_rotations, float* rows,
                       void* stream);

/* Peer-to-peer form of the exchange, for ranks of one NVLink/NVSwitch domain whose receive arenas are mapped
 * into each other's address space (symmetric memory).  cgx_local2j_pack_p2p fuses selection, packing and
 * transport: each selected row is stored straight into the FINAL per-camera tensors of the rank that renders it
 * (plain stores; the local band goes to local memory), behind the rows of lower source ranks
 * (dst[j].first_row), in ascending source index.  It replaces cgx_local2j_pack + the all-to-all + cgx_unpack_rows
 * (gaussian_renderer/__init__.py:612-696).  send_index (optional, with send_row_offset) records the source row
 * of every sent row in local send order for the backward.  cgx_pack_grad_rows_to is the backward's transport:
 * segment r's gradient rows (ncols = 19 or 9 floats each) are stored at seg_rows[r] (host array of device pointers, typically in the
 * source rank's memory).  The caller orders these stores against the readers (stream-ordered barriers). */
typedef struct cgx_peer_camera_dst {
    float* means2D;        /* (n,2) */
    float* rgb;            /* (n,3) */
    float* conic_opacity;  /* (n,4) */
    float* means3D;        /* (n,3) */
    float* scales;         /* (n,3) */
    float* rotations;      /* (n,4) */
    int32_t* radii;        /* (n)   */
    float* depths;         /* (n)   */
    int64_t first_row;     /* first row this rank writes in those arrays */
    float* all_map;        /* (n,5): plane-descriptor form of the record (cgx_local2j_pack_p2p_batched with
                              cgx_exchange_camera.all_map); then means3D / scales / rotations may be null */
} cgx_peer_camera_dst;
int cgx_local2j_pack_p2p(int P, int H, int W, int ws, const float* means2D, const float* rgb,
                         const float* conic_opacity, const float* means3D, const float* scales,
                         const float* rotations, const int32_t* radii, const float* depths,
                         const int32_t* tile_bounds, int avoid_pixel_all2all,
                         const cgx_peer_camera_dst* dst /* host, ws entries */,
                         const int64_t* send_row_offset /* host, ws entries, optional */, int32_t* send_index,
                         void* workspace, size_t workspace_bytes, void* stream);
/* Every camera of a batch in ONE launch of the same kernel (the per-camera loop of
 * gaussian_renderer/__init__.py:612-660 collapsed): cams[k] describes camera k as this rank sends it; each
 * camera's workspace must have been filled by cgx_local2j_count with the same arguments.  All members are 8 bytes
 * wide so that a host can build the array as a plain table of 64-bit words.  Cameras are launched together as
 * long as their participating ranks add up to at most 48 (contiguous cuts give at most cameras + ranks - 1);
 * beyond that the call splits into several launches. */
typedef struct cgx_exchange_camera {
    int64_t P, H, W, ws;
    const float* means2D;
    const float* rgb;
    const float* conic_opacity;
    const float* means3D;
    const float* scales;
    const float* rotations;
    const int32_t* radii;
    const float* depths;
    const int32_t* tile_bounds;            /* device, ws + 1 entries */
    int64_t avoid_pixel_all2all;
    const cgx_peer_camera_dst* dst;        /* host, ws entries */
    const int64_t* send_row_offset;        /* host, ws entries (optional when send_index is null) */
    void* workspace;                       /* device, as left by cgx_local2j_count */
    uint64_t workspace_bytes;
    const float* all_map;                  /* (P,5) or null.  Given (for every camera of the call): the rows carry
                                              this camera's plane descriptors instead of means3D / scales /
                                              rotations, 16 floats per row instead of 21, and land in dst[].all_map */
} cgx_exchange_camera;
int cgx_local2j_pack_p2p_batched(int n_cameras, const cgx_exchange_camera* cams /* host */, int32_t* send_index,
                                 void* stream);
/* The counting stage (cgx_local2j_count) of every camera of a batch in two launches; same reference call site,
 * gaussian_renderer/workload_division.py:721-744 inside the camera loop of gaussian_renderer/__init__.py:612-660.
 * All members are 8 bytes wide; counts: device, ws entries per camera (they may lie anywhere, e.g. in one table). */
typedef struct cgx_count_camera {
    int64_t P, H, W, ws;
    const float* means2D;
    const int32_t* radii;
    const int32_t* tile_bounds;            /* device, ws + 1 entries */
    int64_t avoid_pixel_all2all;
    int32_t* counts;                       /* device, ws entries */
    void* workspace;                       /* device, cgx_local2j_workspace_bytes(P, ws) */
    uint64_t workspace_bytes;
} cgx_count_camera;
int cgx_local2j_count_batched(int n_cameras, const cgx_count_camera* cams /* host */, void* stream);
/* first_segment: the launch works through the rows starting with this segment and wraps around (the result is
 * the same for every value); ranks that pass different values, e.g. (rank + 1) % n_segments, do not all store into
 * the same peer at the same time. */
int cgx_pack_grad_rows_to(int n_segments, float* const* seg_rows, const int64_t* seg_count, int ncols,
                          int first_segment, const float* d_means2D, const float* d_rgb,
                          const float* d_conic_opacity, const float* d_means3D, const float* d_scales,
                          const float* d_rotations, void* stream);
/* cgx_unpack_grad_add for rows of `ncols` floats: 19 = every differentiable column, 9 = means2D | rgb |
 * conic_opacity only (used when no gradient flows back to the 3-D parameters through the exchange), 14 = means2D |
 * rgb | conic_opacity | plane descriptors (5): the (n,5) array takes the place of the means3D argument and the
 * scales / rotations arguments are ignored.  The same three widths hold for cgx_pack_grad_rows_to. */
int cgx_unpack_grad_add_cols(int n_ranges, const int64_t* range_start, const int64_t* range_stop, int ncols,
                             const float* grad_rows, const int32_t* send_index, float* d_means2D, float* d_rgb,
                             float* d_conic_opacity, float* d_means3D, float* d_scales, float* d_rotations,
                             void* stream);

/* Row redistribution by a destination vector: the reference's anchor redistribution
 * (scene/gaussian_model.py:1485-1558 all2all_gaussian_state -- `state[destination == j]` per destination, one list
 * all-to-all per tensor -- driven by redistribute_gaussians :1683-1764) with all tensors packed into one exchange.
 * A travelling row is the concatenation of the row of every tensor, in 4-byte words.
 *   cgx_rows_dest_count  counts[j] = rows with destination j (j < ws), counts[ws] = 1 if some destination lies
 *                        outside [0, ws) (such rows are dropped); leaves per-CTA prefixes in `workspace`.
 *   cgx_rows_pack        stores row i of every tensor at row  dst_first_row[d] + (rows of destination d before i)
 *                        of dst_base[d] (d = destination[i]; rows of `row_words` = sum of words_per_row words):
 *                        ascending local index per destination, as the reference's boolean indexing.  dst_base[d] may
 *                        be a segment owner's send buffer or another GPU's mapped memory (plain stores).
 *   cgx_rows_unpack      splits n received rows back into the tensors.
 * At most 32 destinations and 32 tensors per call; tensors are (rows, words_per_row[t]) arrays of 4-byte words. */
size_t cgx_rows_workspace_bytes(int64_t n, int ws);
int cgx_rows_dest_count(int64_t n, int ws, const int32_t* destination, int32_t* counts, void* workspace,
                        size_t workspace_bytes, void* stream);
int cgx_rows_pack(int64_t n, int ws, const int32_t* destination, int n_tensors, void* const* tensors,
                  const int32_t* words_per_row, uint32_t* const* dst_base, const int64_t* dst_first_row,
                  const void* workspace, void* stream);
int cgx_rows_unpack(int64_t n, const uint32_t* rows, int n_tensors, void* const* tensors,
                    const int32_t* words_per_row, void* stream);

/* Stream-ordered barrier over the ranks of one NVLink/NVSwitch domain (no counterpart in the reference, which
 * synchronises through its collectives).  flag_ptrs: host array of `ws` device pointers, flag_ptrs[r] = an array
 * of at least 32 zero-initialised uint32 words living in rank r's memory and mapped in this process.  Call with
 * the same, strictly increasing epoch on every rank (1, 2, 3, ...).  After the kernel, everything every rank
 * queued before its own call is complete and visible.  The wait is bounded (about 2 s): on expiry the device
 * status word is set (cgx_device_status) and the kernel returns. */
int cgx_peer_barrier(int ws, int rank, uint32_t* const* flag_ptrs, uint32_t epoch, void* stream);
/* The same barrier with the caller's own bound on the wait, in SM clock cycles (0 = the default of about 2 s).
 * A rank that knows its peers are a few microseconds away can fail fast; a test can watch the wait run out:
 * when a peer never signals, the kernel returns after the limit and cgx_device_status reports CGX_ETIMEDOUT. */
int cgx_peer_barrier_limited(int ws, int rank, uint32_t* const* flag_ptrs, uint32_t epoch,
                             unsigned long long wait_limit_cycles, void* stream);

/* ------------------------------------------------------------------ binning */

/* updateTileTouched + InclusiveSum (RAST/cuda_rasterizer/rasterizer_impl.cu:264-288,648).
 * compute_locally: T bytes (bool, row-major Ty x Tx).  Writes tiles_touched u32 (P), the per-block
 * partial sums into workspace, and the total number of (tile, Gaussian) pairs into *num_rendered
 * (device, 1 x u32).  The inclusive offsets themselves are produced by cgx_emit_keys. */
size_t cgx_bin_workspace_bytes(int P);
int cgx_bin_count_scan(int P, int W, int H, const int32_t* radii, const float* means2D,
                       const uint8_t* compute_locally, uint32_t* tiles_touched, uint32_t* num_rendered,
                       void* workspace, size_t workspace_bytes, void* stream);
/* The same stage, also reducing the depths of the splats that will emit keys: num_rendered3[0] = pairs,
 * [1] / [2] = smallest / largest bit pattern of their (positive) depths (0xffffffff / 0 when there are none).  The
 * caller reads all three in the host read it makes anyway; the leading bits the two patterns share are equal in
 * every sort key, which is what cgx_sort_pairs_pingpong's low_bits wants:
 * low_bits = 32 - clz(min ^ max)  (at least 1). */
int cgx_bin_count_scan_depths(int P, int W, int H, const int32_t* radii, const float* means2D, const float* depths,
                              const uint8_t* compute_locally, uint32_t* tiles_touched, uint32_t* num_rendered3,
                              void* workspace, size_t workspace_bytes, void* stream);

/* duplicateWithKeys (RAST/cuda_rasterizer/rasterizer_impl.cu:74-117): writes point_offsets u32 (P)
 * (inclusive sum, as the reference's GeometryState::point_offsets), keys u64 (R) =
 * (tile << 32) | bits(depth), values u32 (R) = Gaussian index, emission order y-major then x over the
 * locally computed tiles of the Gaussian's rectangle.  capacity = number of pairs keys/values can hold
 * (normally the total written by cgx_bin_count_scan); pairs beyond it are dropped, never written.
 * workspace: the buffer cgx_bin_count_scan filled for the same inputs. */
int cgx_emit_keys(int P, int W, int H, const int32_t* radii, const float* means2D, const float* depths,
                  const uint32_t* tiles_touched, const uint8_t* compute_locally,
                  uint32_t* point_offsets, uint64_t* keys, uint32_t* values, int64_t capacity,
                  const void* workspace, void* stream);

/* cub::DeviceRadixSort::SortPairs call site (RAST/cuda_rasterizer/rasterizer_impl.cu:679-684):
 * stable ascending sort of (key, value) pairs on key bits [0, end_bit), 8 bits per pass.  keys_in/values_in are
 * clobbered (used as ping-pong buffers); the result is in keys_out/values_out.  Per pass: per-tile digit
 * histograms kept on chip, a scan of the digit rows, and a stable scatter; no kernel waits for another CTA. */
size_t cgx_sort_workspace_bytes(int64_t n);
int cgx_sort_pairs(int64_t n, int end_bit, uint64_t* keys_in, uint32_t* values_in, uint64_t* keys_out,
                   uint32_t* values_out, void* workspace, size_t workspace_bytes, void* stream);

/* The same sort for a caller that owns both buffers and can choose where its pairs start (same call site: the
 * reference's BinningState holds both the unsorted and the sorted arrays, rasterizer_impl.cu:188-205).  The pairs
 * start in (keys_a, values_a); the result lands in (keys_a, values_a) when the number of passes is even and in
 * (keys_b, values_b) when it is odd, so no copy is ever needed.
 * low_bits (1..32; 32 = plain sort): the caller asserts that bits [low_bits, 32) of every key are equal (for
 * (tile << 32 | depth) keys: the sign, the leading exponent bits ... that all depths of a view share; see
 * cgx_bin_count_scan_depths).  Equal bits cannot change a stable order, so they are squeezed out of the digits:
 * passes = cgx_sort_passes(end_bit - (32 - low_bits)), often one fewer.  The keys themselves are moved unchanged.
 * wait_limit_cycles: only used by the test-only one-sweep variant (bound of its look-back wait in SM clock cycles,
 * 0 = default of about 0.14 s). */
int cgx_sort_passes(int end_bit);
int cgx_sort_pairs_pingpong(int64_t n, int end_bit, int low_bits, uint64_t* keys_a, uint32_t* values_a,
                            uint64_t* keys_b, uint32_t* values_b, void* workspace, size_t workspace_bytes,
                            unsigned long long wait_limit_cycles, void* stream);


/* No counterpart in the reference.  Same sort as cgx_sort_pairs for callers that may not allocate device
 * memory (an engine with a memory budget fixed at start-up, a plugin whose host has frozen the CUDA pools, a
 * latency path that must stay away from the allocator): the digit tables live in a fixed array inside the
 * loaded module, so the call takes no workspace and allocates nothing.
 *   - at most cgx_sort_pairs_static_max() = 4,194,304 pairs; larger n returns CGX_ENOMEM and
 *     cgx_last_cuda_error() explains;
 *   - the first call on each device looks up the array's device address (with that device current); make
 *     that first call before starting any stream capture;
 *   - all calls on a device share the one array.  Nothing in it has to start at zero (every pass rewrites
 *     the entries it reads), but two sorts that overlap on the GPU (different streams) corrupt each other:
 *     keep calls on one device ordered. */
int64_t cgx_sort_pairs_static_max(void);
int cgx_sort_pairs_static(int64_t n, int end_bit, uint64_t* keys_in, uint32_t* values_in, uint64_t* keys_out,
                          uint32_t* values_out, void* stream);

/* cudaMemset + identifyTileRanges (RAST/cuda_rasterizer/rasterizer_impl.cu:122-144,687-695):
 * ranges uint2 (T): [start, end) into the sorted list; empty tiles get (0,0). */
int cgx_tile_ranges(int64_t n, int T, const uint64_t* keys_sorted, uint32_t* ranges, void* stream);

/* ------------------------------------------------------------------ blending */

/* RenderGaussiansCUDA -> renderForward -> renderCUDA (RAST/rasterize_points.cu:276-364,
 * RAST/cuda_rasterizer/rasterizer_impl.cu:699-725, RAST/cuda_rasterizer/forward.cu:264-486).
 * Writes every pixel of every image output (zeros in tiles that are not computed locally) and zero-fills
 * out_observe before accumulating.  records: scratch for P 64-byte packed records (see
 * cgx_render_records_bytes), kept by the caller for the backward; when `radii` is given, records of
 * Gaussians with radius <= 0 (never listed in any tile) are left unwritten.
 *   -> final_T f32 (H*W), n_contrib u32 (H*W), n_contrib2loss u32 (H*W), out_color (3,H,W),
 *      out_observe int32 (P), out_all_map (5,H,W), out_plane_depth (1,H,W),
 *      and the per-tile statistics of cgx_tile_stats (n_render, n_consider, n_contrib: int32 (T)),
 *      reduced in the kernel's epilogue.                                                         */
size_t cgx_render_records_bytes(int P);
int cgx_render_fwd(int P, int W, int H, float tanfovx, float tanfovy, const uint32_t* ranges,
                   const uint32_t* point_list, const int32_t* radii /* optional */, const float* means2D, const float* rgb, const float* all_map,
                   const float* conic_opacity, const uint8_t* compute_locally, const float* bg, int render_geo,
                   void* records, float* final_T, uint32_t* n_contrib, uint32_t* n_contrib2loss,
                   float* out_color, int32_t* out_observe, float* out_all_map, float* out_plane_depth,
                   int32_t* n_render, int32_t* n_consider, int32_t* n_contrib_tile, void* stream);

/* get_n_render + reduce_data_per_block x2 (RAST/cuda_rasterizer/rasterizer_impl.cu:219-262,730-752):
 * per-tile int32 (T) outputs; every element written. */
int cgx_tile_stats(int W, int H, const uint32_t* ranges, const uint32_t* n_contrib_px,
                   const uint32_t* n_contrib2loss_px, const uint8_t* compute_locally,
                   int32_t* n_render, int32_t* n_consider, int32_t* n_contrib, void* stream);

/* RenderGaussiansBackwardCUDA -> renderBackward -> renderCUDA(bwd) (RAST/rasterize_points.cu:366-441,
 * RAST/cuda_rasterizer/rasterizer_impl.cu:850-932, RAST/cuda_rasterizer/backward.cu:324-567,643-696),
 * including the (P,2,2)+(P,1) -> (P,4) repack of rasterize_points.cu:428-436.  Zero-fills and then
 * accumulates:  dL_dmeans2D (P,2), dL_dmeans2D_abs (P,3), dL_dconic_opacity (P,4), dL_drgb (P,3),
 * dL_dall_map (P,5).  records: the buffer cgx_render_fwd filled for the same inputs. */
int cgx_render_bwd(int P, int W, int H, float tanfovx, float tanfovy, const uint32_t* ranges,
                   const uint32_t* point_list, const float* bg, const void* records,
                   const float* all_map_pixels, const float* final_T, const uint32_t* n_contrib,
                   const uint8_t* compute_locally, const float* dL_dcolor, const float* dL_dout_all_map,
                   const float* dL_dout_plane_depth, int render_geo,
                   float* dL_dmeans2D, float* dL_dmeans2D_abs, float* dL_dconic_opacity, float* dL_drgb,
                   float* dL_dall_map, int walk, void* stream);

/* How the backward pass chooses its walk.  cgx_render_fwd leaves, behind the P records of its `records` buffer,
 * cgx_render_density_words() 64-bit counters: pairs (pixels that passed the alpha test, visits of a Gaussian to an
 * 8x4 pixel block), spread over slots.  walk = 0: cgx_render_bwd queues both of its kernels and the one the
 * counters do not call for returns at once (no host read).  A caller that has the counters on the host anyway
 * (copied behind the forward pass; by the time of the backward pass they have usually arrived) sums the pairs and
 * passes walk = 2 (every pixel looks at every visit) when pixels > cgx_render_dense_threshold() * visits, else
 * walk = 1 (every pixel walks its own list): one launch instead of two. */
int cgx_render_density_words(void);
int cgx_render_dense_threshold(void);

/* ------------------------------------------------------------------ diagnostics */

/* Host-synchronous.  Waits for `stream`, reads and clears the device status word that kernels set when a
 * bounded wait (blending mbarriers, peer barrier, the sort's look-back) gives up (0 = ok, CGX_ETIMEDOUT otherwise).  Replaces the reference's debug-mode
 * synchronise-and-throw (RAST/cuda_rasterizer/auxiliary.h:220-227); nothing ever traps. */
int cgx_device_status(int* status_host, void* stream);

/* The same status words without waiting: queues their copies on `stream` into status_pinned_host4[0..2]
 * (page-locked host memory: blending kernels, peer barrier, sort look-back; [3] is reserved and set to 0).  The
 * caller looks at them after a synchronisation it performs anyway (0 = ok); the words are not cleared
 * (cgx_device_status clears them). */
int cgx_device_status_async(int* status_pinned_host4, void* stream);

/* Copies n_words32 32-bit words from device memory to page-locked host memory with a one-CTA kernel that stores
 * through the host mapping (CGX_EINVAL for pageable memory or misaligned pointers).  For the few words a host waits
 * for inside a step (the pair count, the exchange's size table, the status words): a copy-engine transfer of them
 * queues behind bulk device-to-host copies of other streams, a kernel does not.  The reference reads its pair
 * count with a blocking cudaMemcpy (RAST/cuda_rasterizer/rasterizer_impl.cu:652-653). */
int cgx_post_words(const void* src_device, void* dst_host_pinned, int n_words32, void* stream);


#ifdef __cplusplus
}
#endif
#endif /* CGX_RASTER_H */
