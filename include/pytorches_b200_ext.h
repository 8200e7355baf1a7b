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
 * Tells the plugin that the host has put work of its own on `device`'s stream (the one above).
 * The plugin lets a full-tensor reduction START while the previous one it enqueued is still in its
 * last microseconds (the ordered combine of the block sums, the exchange with peer GPUs), when it
 * enqueued nothing else between the two and their buffers are disjoint; results and their order are
 * unaffected. It cannot see a kernel the host launches on the stream directly, so after doing that
 * the host calls this once and the next reduction is launched the ordinary way. Event records,
 * event waits and copies need no call: they separate the kernels around them by themselves.
 * Replaces nothing in the reference.
 */
void pytorches_b200_stream_touched(uint32_t device);

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
 * The result is bit-identical to SUM_AXIS over a 1-D tensor of the same data. Returns a PtStatus;
 * after a failure last_error() of the vtable says why. The calling thread's current CUDA device is
 * the same after the call as before it.
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
 * pytorches_b200_peer_mean(device, x, n, n_total, seq, out) is the mean of the whole tensor of
 * n_total elements: the sum as above, divided in the same kernel by n_total as an f32. Same bits as
 * the reference's mean over the gathered per-rank sums, which is SUM_AXIS then DIV by a scalar tensor
 * holding the element count (crates/core/src/lib.rs:662-670).
 *
 * `seq` numbers the reductions of the group: every rank must pass the same value for the same
 * reduction and a different one for the next (a counter). All ranks must call in the same order. If
 * a peer's result does not arrive within wait_ms the kernel gives up, nothing hangs, and the next
 * blocking vtable call on the device returns PT_STATUS_INTERNAL once. All return a PtStatus.
 *
 * `x` may be any f32 device pointer of that GPU (4-byte aligned), not only the start of a plugin
 * buffer: a pointer that is not 16-byte aligned takes the kernels' narrow-load forms, with the same
 * result. `out` must be aligned to its type (4 bytes, 8 for argmax). Other alignments are refused
 * with PT_STATUS_INVALID_ARGUMENT.
 */
int32_t pytorches_b200_peer_export(uint32_t device, void *handle_out);
int32_t pytorches_b200_peer_attach(uint32_t device, uint32_t rank, uint32_t world, const void *handles, uint32_t wait_ms);
int32_t pytorches_b200_peer_reduce(uint32_t device, uint32_t kind, const float *x, uint64_t n, int64_t first_index, uint64_t seq, void *out);
int32_t pytorches_b200_peer_mean(uint32_t device, const float *x, uint64_t n, uint64_t n_total, uint64_t seq, float *out);

/*
 * The sum (mean != 0: the mean) of the whole tensor with the BITS OF THE UNSPLIT SUM, for shards that
 * are runs of whole 65536-element blocks of it (first_index a multiple of 65536, and n too unless the
 * shard ends the tensor). The reference adds a long row as a chain of 65536-element block sums in
 * block order (plugins/cpu/src/reduce.rs:110-131); here every GPU's block sums travel to every rank's
 * window (one self-validating word each, plain peer stores as they are produced) and every rank runs
 * that chain over all of them, so a tensor reduced on 1, 2, 4 or 8 GPUs gives the same bits, those of
 * the reference on the unsplit tensor, as its rule for split execution asks
 * (tests/diff/test_placement.py:135-144). n_total is at most 2^30 elements (16384 blocks); `x` must be
 * 16-byte aligned. Everything else (seq, bounded waits, error reporting) as for peer_reduce. A replayed
 * PT_B200_CALL_PEER_REDUCE names it with op = 4 (sum) or 5 (mean), ints[0] = first_index, ints[1] = n_total.
 */
int32_t pytorches_b200_peer_sum_unsplit(uint32_t device, const float *x, uint64_t n, uint64_t first_index, uint64_t n_total, uint32_t mean,
                                        uint64_t seq, float *out);

/*
 * Where the time of the sharded reductions goes (a diagnostic: set PYTORCHES_B200_PEER_TRACE=1 in the
 * environment before the windows are attached; off by default because the extra stores were measured
 * to disturb multi-GPU runs). Every reduction with an in-kernel exchange then leaves device-clock
 * readings (nanoseconds, %globaltimer) in a per-device buffer, in record
 * (seq % 0xfffffffe + 1) % 64 of sixteen words: [1] this GPU's own part is complete, [2] every rank's
 * part has arrived, [3] the result is written; a sum in unsplit order also leaves [13], how many bulk
 * copies of the block sums its combiner needed (a count, not a time). The other words are unused.
 * [2] - [1] is the wait for the slowest peer (skew between the GPUs plus NVLink latency), [3] - [2]
 * the work left after the last arrival. This call synchronizes the device's stream and copies the 64
 * records (64 x 16 uint64) to `records_out`. Replaces nothing in the reference.
 */
int32_t pytorches_b200_peer_trace(uint32_t device, uint64_t *records_out);

/*
 * The same for a small vector result: the sum over the leading dimension of a [rows_total, cols]
 * tensor whose rows are split over the ranks, e.g. the bias gradient the reference core computes by
 * SUM_AXIS(0) when it reduces a broadcast gradient back to the bias's shape
 * (crates/core/src/lib.rs:578-591). `x` = this rank's [rows, cols] rows (rows may differ between
 * ranks, may be 0), `out` = cols f32 values: the per-rank column sums, exchanged through the windows
 * (one self-validating word per element) and added in rank order on every rank, the bits SUM_AXIS(0)
 * gives over the gathered [world, cols] tensor of per-rank sums. cols is at most 4096 (16 KiB of
 * results); larger results are refused with PT_STATUS_INVALID_ARGUMENT and belong to a collective
 * library. `seq` counts in the same sequence as the scalar reductions.
 */
int32_t pytorches_b200_peer_sum_axis0(uint32_t device, const float *x, uint64_t rows, uint64_t cols, uint64_t seq, float *out);

/*
 * Replay of a recorded call list. The reference core issues one `execute` per tensor op, each with
 * an `alloc` for its result before and `free`s as tensors die (crates/core/src/lib.rs:331-370); a
 * training or benchmark step repeats the same list of calls every time. This entry point takes such
 * a list once and issues it `repeats` times from native code, call for call through the same alloc,
 * free and execute the vtable exposes, so that a host written in a slow language does not become the
 * bottleneck when the ops run for tens of microseconds. It replaces nothing in the reference (whose
 * core is native code already); the Python host in this repository records its own op sequences
 * with it.
 *
 * A call is one of: PT_B200_CALL_EXECUTE (`op`, `ints` = the OpAttrs, `in`/`out` = the descriptors),
 * PT_B200_CALL_ALLOC (ints[0] = bytes, ints[1] = slot: the block is kept in that slot),
 * PT_B200_CALL_FREE (ints[1] = slot), PT_B200_CALL_PEER_REDUCE (`op` = kind 0 sum, 1 max, 2 argmax,
 * 3 mean; in[0] = this rank's shard as a 1-D tensor, out[0] = the result; ints[0] = first_index,
 * ints[1] = the whole tensor's element count for a mean; `seq` is first_seq for the first such call
 * and counts up from there across calls and repeats). An operand names its memory either directly
 * (`slot` < 0, `data` = device pointer, which must stay valid) or as the block currently in `slot`.
 * Blocks still in a slot when a pass over the list ends are freed, as when a host drops the results
 * of a step. Stops at the first call that fails and returns its PtStatus (last_error() says why).
 */
enum { PT_B200_CALL_EXECUTE = 0, PT_B200_CALL_ALLOC = 1, PT_B200_CALL_FREE = 2, PT_B200_CALL_PEER_REDUCE = 3 };

typedef struct PtB200Operand {
    void *data;
    int32_t slot;
    uint32_t dtype;
    uint32_t ndim; /* at most 8 */
    uint32_t reserved;
    uint64_t shape[8];
    uint64_t strides[8];
} PtB200Operand;

typedef struct PtB200Call {
    uint32_t kind;
    uint32_t op;
    int64_t ints[4];
    uint32_t n_in, n_out; /* at most 2 each */
    PtB200Operand in[2];
    PtB200Operand out[2];
} PtB200Call;

int32_t pytorches_b200_replay(uint32_t device, const PtB200Call *calls, uint32_t n_calls, uint32_t repeats, uint64_t first_seq);

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
