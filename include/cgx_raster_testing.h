/* Test-only switches of libcgx_raster.so: NOT part of the drop-in boundary.
 *
 * They select between kernel variants that produce the same results, for A/B timing and for tests that check
 * exactly that equality.  They are process-wide and not thread-safe; production callers never touch them, so the
 * library's entry points in cgx_raster.h stay free of caller-visible mutable state. */
#ifndef CGX_RASTER_TESTING_H
#define CGX_RASTER_TESTING_H
#ifdef __cplusplus
extern "C" {
#endif

/* Scatter strategy of the sort, for A/B timing and tests: -1 (default) chooses by size (unstaged while both
 * ping-pong buffers fit in L2, staged above), 0 always staged, 1 always unstaged.  Results are identical. */
int cgx_set_sort_variant(int variant);

/* A/B switches of the blending kernels (default 1 = culling only), for timing and tests:
 *   bit 0  per-warp culling of each batch before blending (forward and backward; results bit-identical);
 *   bit 1  backward: the per-channel "accumulated behind" recurrences contracted with the pixel cotangent
 *          (faster; leaves the 1e-3 gradient parity band on pixels whose plane-depth cotangent blows up);
 *   bit 2  backward: visits with one or two contributing pixels issue their atomics directly (measured slower). */
int cgx_set_render_variant(int variant);

#ifdef __cplusplus
}
#endif
#endif
