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

/* Pass structure of the sort, for A/B timing and tests: -1 (default) three kernels per pass (histogram, scan,
 * scatter; the scatter staged through shared memory above 4 M pairs, unstaged below); 0 always staged; 1 always
 * unstaged; 2 one kernel per pass with bounded look-back over published tile counts ("one-sweep": measured slower
 * on B200 at these sizes, 0.54 ms against 0.37 ms for 4.26 M pairs of 45 bits).  Results are identical. */
int cgx_set_sort_variant(int variant);

/* A/B switch of the blending kernels (default 1):
 *   bit 0  per-warp culling of each batch before blending (forward and backward);
 *   bit 1  always the reference-shaped walk (every lane looks at every surviving Gaussian; butterfly reduction of
 *          the gradient terms in the backward);
 *   bit 2  always the two-phase walk (every lane walks only its own contributors; gradient terms staged in shared
 *          memory and summed per Gaussian).
 * With neither bit 1 nor bit 2 the walk follows the density the forward pass measures (pixels reached per visit):
 * per chunk of visits in the forward, per launch in the backward.  Forward outputs are bit-identical across the
 * variants; gradients differ by the order of their sums. */
int cgx_set_render_variant(int variant);

#ifdef __cplusplus
}
#endif
#endif
