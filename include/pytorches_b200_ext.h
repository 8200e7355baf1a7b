/*
 * Entry points pytorches_plugin_b200.so exports besides `pytorches_plugin_entry`.
 *
 * The plugin vtable (pytorches_plugin_abi.h) is everything the reference core calls. These extra
 * symbols exist for hosts that need to see a little further than ABI 4 lets them: to time work on
 * the device, to interoperate with other CUDA code in the same process, and to prove that work ran
 * on the GPU. The reference lists the underlying needs as open questions of its ABI
 * (docs/plugin-abi.md:278-282, "Streams and events", "Pointer export"); none of these symbols is
 * required to use the plugin through the vtable.
 */
#ifndef PYTORCHES_B200_EXT_H
#define PYTORCHES_B200_EXT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * The CUDA stream (a `cudaStream_t`) that is the implicit in-order stream of `device`
 * (docs/plugin-abi.md:144-158), or NULL if the device does not exist. Everything the vtable enqueues
 * for that device runs on it, so CUDA events recorded on it bracket the plugin's work, and a
 * collective enqueued on it is ordered with the plugin's kernels. The stream lives as long as the
 * process. Replaces nothing in the reference: ABI 4 has no stream handles.
 */
void *pytorches_b200_stream(uint32_t device);

/*
 * Number of CUDA kernels this library has launched since it was loaded (all devices, all threads).
 * Copies are not counted. Replaces nothing in the reference.
 */
uint64_t pytorches_b200_kernel_launches(void);

/*
 * Sum of the n f32 values at `x` into `out[0]`, for hosts that cannot allocate device memory when
 * they call: a process that handed the whole GPU to its own memory pool at start-up (a serving
 * process, another framework's caching allocator) has nothing left for a library to allocate from,
 * and a host with a latency bound may forbid allocator calls on its hot path because they can stall
 * every stream of the device. The vtable's SUM_AXIS takes its inter-pass scratch from the plugin's
 * allocator; this entry point keeps that scratch in a fixed 256 KiB array inside the library
 * instead (every GPU that loads the library holds the array until the process exits) and calls no
 * allocation or free routine of CUDA, of this plugin, or of any other library.
 *
 * It has no counterpart in the reference, whose ABI always lets a plugin allocate.
 *
 *   device  index of the GPU that `x` and `out` live on
 *   x, out  device pointers owned by the caller (any memory of that GPU, not only the plugin's)
 *   n       element count; at most 2^32 (the array holds one partial sum per 65536 elements).
 *           Larger n is refused with PT_STATUS_INVALID_ARGUMENT and a message naming the limit,
 *           readable through the vtable's last_error(); nothing is launched.
 *   stream  the cudaStream_t to enqueue on (NULL is CUDA's default stream); the call returns
 *           once the kernels are queued, like the vtable's execute
 *
 * The result is bit-identical to SUM_AXIS over a 1-D tensor of the same data. Returns a PtStatus.
 *
 * The first call on each device looks up the array's address on that device (one
 * cudaGetSymbolAddress); make that first call outside any stream capture. All calls on one GPU share
 * the one array: two calls whose kernels can overlap on the GPU (different streams, no ordering
 * between them) race on it and both results are undefined. Calls ordered on one stream are safe,
 * and no call depends on what an earlier one left in the array: each overwrites the slots it reads.
 */
int32_t pytorches_b200_sum_noalloc(uint32_t device, const float *x, uint64_t n, float *out, void *stream);

/*
 * Reductions over a tensor whose rows are split across several GPUs, one process per GPU, with the
 * exchange of the per-GPU results done INSIDE the reduction kernel over peer memory instead of by a
 * collective library. The reference has no multi-GPU execution of one op (its planner places whole
 * layers, crates/core/src/strategy.rs:221-326, and moves tensors through host memory,
 * crates/core/src/lib.rs:535-542), so these replace nothing in it.
 *
 * Each process owns a small "window" of device memory per GPU. pytorches_b200_peer_export creates and
 * zeroes this device's window and writes its 64-byte CUDA IPC handle to `handle_out`; the host
 * exchanges the handles between the ranks by whatever means it has (the Python host uses
 * torch.distributed); pytorches_b200_peer_attach(device, rank, world, handles, wait_ms) then maps the
 * other ranks' windows (`handles` = world x 64 bytes in rank order, this device's own at index `rank`;
 * world <= 8; wait_ms = how long a kernel waits for its peers, 0 = 2000).
 *
 * pytorches_b200_peer_reduce(device, kind, x, n, first_index, seq, out) enqueues, on the device's
 * stream, the reduction of this rank's n f32 values at `x` AND the combination with every other
 * rank's result: kind 0 = sum (f32 to out), 1 = max (f32), 2 = argmax (i64: position in the whole
 * tensor, `first_index` being where this rank's shard starts in it). The kernel that finishes the
 * local reduction stores the result with plain peer stores into a slot of EVERY rank's window, waits
 * (bounded) until its own window holds all ranks' results, combines them in rank order and writes
 * `out`; every rank ends with the same bits, those the vtable ops give when they combine the gathered
 * per-rank results (SUM_AXIS / MAX_AXIS / ARGMAX_COMBINE over a [world, ...] tensor).
 *
 * `seq` numbers the reductions of the group: every rank must pass the same value for the same
 * reduction and a different one for the next (a counter). All ranks must call in the same order. If
 * a peer's result does not arrive within wait_ms the kernel gives up, nothing hangs, and the next
 * blocking vtable call on the device returns PT_STATUS_INTERNAL once. All return a PtStatus.
 */
int32_t pytorches_b200_peer_export(uint32_t device, void *handle_out);
int32_t pytorches_b200_peer_attach(uint32_t device, uint32_t rank, uint32_t world, const void *handles, uint32_t wait_ms);
int32_t pytorches_b200_peer_reduce(uint32_t device, uint32_t kind, const float *x, uint64_t n, int64_t first_index, uint64_t seq, void *out);

/*
 * Failure-path self test. The staged reduction kernels wait for their asynchronous copies with a
 * bounded number of tries; if a wait ever ran out they would record it in a host-visible status word
 * and the next blocking vtable call (synchronize, copy_to_host) would return PT_STATUS_INTERNAL
 * instead of a wrong result (docs/plugin-abi.md:155-156, deferred failures). This entry point enqueues,
 * on `stream`, a tiny kernel whose wait is certain to run out (it waits for bytes nobody sends, for a
 * few thousand tries: milliseconds) and that reports it through the same word. The GPU neither hangs
 * nor faults. After it, exactly one blocking call on that device reports the error; later calls work.
 * Replaces nothing in the reference. Returns a PtStatus for the enqueue itself.
 */
int32_t pytorches_b200_selftest_expired_wait(uint32_t device, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* PYTORCHES_B200_EXT_H */
