// What the LinearCuda / Conv2dCuda shims tell the data-parallel exchange (ddp_b200.cpp): "the parameter deltas at this
// device address have just been launched on the legacy default stream". When a DDPSequential registered that tensor,
// the call marks it ready, and the bucket that it completes starts its allreduce on the exchange's own stream while
// the backward pass of the earlier layers goes on. Without a DDPSequential in the process the call does nothing.
#pragma once
void ddp_b200_deltas_ready(const float *device_ptr);
// The tcgen05 kernels bound every device-side wait; a wait that ran out leaves a non-zero status word instead of a hung
// GPU. Shims call this where they synchronise with the device anyway; it raises LOG(ERROR) when the word is set.
void tagi_b200_raise_on_kernel_abort();
