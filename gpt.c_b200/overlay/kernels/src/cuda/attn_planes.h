// Hand-off between the Linear adapter and the attention adapter of the overlay: when a Linear
// forward looks like the fused QKV projection (out_features == 3 * in_features, head size 64),
// it also emits its result as the bf16 planes the attention kernels read and offers them here;
// the attention forward that receives the same tensor takes them and skips its own split pass.
// One slot only.  An offer that nobody takes is released by the next offer, by the attention adapter when
// it runs a head size the planes are not made for, or by the allocator when the tensor it belongs to is
// freed: the stream-ordered pool hands a freed address to the next tensor of the same size, so an offer
// must not outlive its tensor.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// `planes` was allocated with alloc_cuda and holds `bytes` bytes of planes for the tensor at `y`.
void overlay_planes_offer(const float *y, void *planes, size_t bytes);
// Returns the planes offered for `y` when they hold exactly `bytes` bytes (ownership passes to the
// caller, who releases them with free_cuda), else NULL.
void *overlay_planes_take(const float *y, size_t bytes);
// Releases the pending offer when it belongs to the tensor at `y` (called by free_cuda for every pointer
// it frees) or, with y == NULL, whatever is pending.
void overlay_planes_forget(const void *y);

#ifdef __cplusplus
}
#endif
