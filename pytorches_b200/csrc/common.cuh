// Internal declarations shared by the plugin's translation units: launch plumbing, exact integer
// division for index math, and the launcher entry points the boundary (plugin.cu) dispatches to.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstddef>
#include <cstdint>

namespace b200 {

// Coalesced dims a kernel accepts (after dropping size-1 dims and merging contiguous neighbours).
constexpr int MAX_DIMS = 8;

// Number of kernels launched by this library since load (reported through the extension API).
extern std::atomic<uint64_t> g_kernel_launches;

// B200 has 148 SMs; grids of persistent kernels are sized from the queried count at run time.
int sm_count(int device);

// Stores `msg` as the calling thread's last error (what the vtable's last_error() returns).
void set_last_error(const char *msg);

// Tells the boundary that something it did not enqueue itself went onto `device`'s stream: the next
// reduction is then launched the ordinary way (see LaunchChain).
void note_foreign_enqueue(int device);

// Exact floor division by a runtime constant. For 32-bit operands: Lemire's method,
// floor(n/d) = hi64(ceil(2^64/d) * n) for every n, d < 2^32 (d > 1). For 64-bit operands the
// hardware-emulated division is used; that path only runs for tensors of 2^32 or more work items.
template <typename I> struct Divider;
template <> struct Divider<uint32_t> {
    uint64_t magic;
    uint32_t d;
    Divider() : magic(0), d(1) {}
    explicit Divider(uint64_t d_) : magic(d_ > 1 ? UINT64_MAX / d_ + 1 : 0), d((uint32_t)d_) {}
    __device__ __forceinline__ void divmod(uint32_t n, uint32_t &q, uint32_t &r) const {
        q = d == 1 ? n : (uint32_t)__umul64hi(magic, (uint64_t)n);
        r = n - q * d;
    }
};
template <> struct Divider<uint64_t> {
    uint64_t d;
    Divider() : d(1) {}
    explicit Divider(uint64_t d_) : d(d_) {}
    __device__ __forceinline__ void divmod(uint64_t n, uint64_t &q, uint64_t &r) const {
        q = n / d;
        r = n - q * d;
    }
};

// One coalesced dimension of an elementwise op: its size and each operand's element stride.
struct EwDim {
    uint64_t size;
    uint64_t stride[2];
};

// Elementwise problem after host-side coalescing (reference: plugins/cpu/src/ew.rs:22-43).
struct EwProblem {
    int nd = 0;          // coalesced dims, outermost first; 0 means a single element
    EwDim dim[MAX_DIMS];
    uint64_t n = 1;      // output elements
};

// ---- launchers (each enqueues on `s` and returns the CUDA error of the launch) --------------------
cudaError_t launch_unary(uint32_t op, const float *x, float *out, const EwProblem &p, cudaStream_t s);
cudaError_t launch_binary(uint32_t op, const float *a, const float *b, float *out, const EwProblem &p, cudaStream_t s);
cudaError_t launch_axpy(const float *a, const float *b, float *out, float alpha, uint64_t n, cudaStream_t s);
cudaError_t launch_fill(float *out, uint64_t n, float v, cudaStream_t s);
cudaError_t launch_randn(float *out, uint64_t n, uint64_t seed, cudaStream_t s);
cudaError_t launch_rand_uniform(float *out, uint64_t n, uint64_t seed, float lo, float scale, uint64_t first, cudaStream_t s);
cudaError_t launch_matmul(const float *a, uint64_t ars, uint64_t acs, const float *b, uint64_t brs, uint64_t bcs,
                          float *c, uint64_t m, uint64_t n, uint64_t k, cudaStream_t s);

// Reductions over the middle axis of a contiguous (outer, len, inner) tensor. `scratch` must hold
// reduce_scratch_bytes(...) bytes (0 means none is needed); it is global memory the kernels use for
// per-block partial results between their two passes.
// SUM and MAX write f32 values to out_v, ARGMAX i64 positions to out_i, MAX_ARGMAX both; positions
// get idx_offset added (the shard's first row when the axis is split over devices).
enum ReduceKind : int { REDUCE_SUM = 0, REDUCE_MAX = 1, REDUCE_ARGMAX = 2, REDUCE_MAX_ARGMAX = 3 };

// The cross-GPU step of a reduction whose input is split over several GPUs (one process each): what a
// kernel needs to hand its GPU's result to every peer and to collect theirs. Every rank owns a small
// "window" of device memory that all ranks have mapped (CUDA IPC); rank r's result for the reduction
// numbered `epoch` goes, as plain peer stores over NVLink, into slot r of EVERY rank's window, so that
// each rank then finds all results in its OWN memory and combines them in rank order. world == 0
// means "no cross-GPU step".
constexpr int PEER_MAX_RANKS = 8;
struct PeerXchg {
    unsigned long long *window[PEER_MAX_RANKS];  // rank r's window as mapped in this process; [rank] is local memory
    int world;
    int rank;
    uint32_t epoch;          // never 0; the same on every rank for the same reduction
    uint32_t wait_ms;        // how long to wait for the peers before giving up
    float divide_by;         // a sum's combined result is divided by this when it is not 0 (mean = sum / count)
    // A sum "in unsplit order": the shards are whole 65536-element blocks of one tensor of blocks_total
    // blocks, this rank's first being block0. Every worker then stores its block sum into EVERY rank's
    // window and every rank's combiner chains all blocks_total sums in block order: the result has the
    // bits of the sum over the unsplit tensor. blocks_total == 0: per-rank results combined in rank order.
    uint32_t block0;
    uint32_t blocks_total;
    unsigned long long *trace;  // this device's trace records (see peer_trace in reduce.cu); ordinary device memory, not part of a window
};
// Window management (one window per device of this process). `handle` is a 64-byte CUDA IPC handle.
cudaError_t peer_window_export(int device, void *handle, cudaStream_t s);
cudaError_t peer_window_attach(int device, uint32_t rank, uint32_t world, const void *handles, uint32_t wait_ms);
bool peer_window_for(int device, uint64_t seq, PeerXchg *px);
cudaError_t peer_trace_read(int device, unsigned long long *out, cudaStream_t s);

size_t reduce_scratch_bytes(ReduceKind kind, uint64_t outer, uint64_t len, uint64_t inner, int device);

// What the boundary remembers about the last thing it enqueued on a device's stream, so that a
// reduction can be allowed to start while the previous one is still finishing. A full-tensor reduction
// over a long row ends in one combiner CTA (ordered chain over the block sums, the exchange with peer
// GPUs); its worker CTAs are long done by then. Such a kernel signals early that dependents may
// launch, and if the NEXT thing enqueued is again such a reduction with buffers disjoint from this
// one's, it is launched with programmatic stream serialization: its workers stream while this one's
// combiner finishes. Ordering is kept where it matters: a combiner lets the kernel after its own
// start only when the combiner two launches back has finished, and finishes only after the kernel
// before its own has completed. So at most three such kernels are at work (one chaining, one
// streaming, one starting), they complete in launch order, and a launch must be disjoint from the
// two before it. Any other kind of work is launched normally and starts after everything before it
// has completed; `tail_open` is false after anything else.
struct LaunchChain {
    struct Open {
        const char *in_lo = nullptr, *in_hi = nullptr;  // an unfinished reduction's input range
        const void *out[2] = {nullptr, nullptr};        // and its outputs
    };
    bool tail_open = false;  // the newest launch on the stream is such a reduction
    Open last, before_last;  // it, and the one launched before it if that one may be unfinished too (else all null)
};

// With `px` (only for outer == inner == 1): the result written is the combination over all ranks, in
// rank order, of every rank's result; MAX_ARGMAX then needs both outputs, ARGMAX is not offered.
// `chain` (may be null: no overlap) is read to decide how to launch and updated to describe this launch.
cudaError_t launch_reduce(ReduceKind kind, const float *x, uint64_t outer, uint64_t len, uint64_t inner, float *out_v,
                          int64_t *out_i, int64_t idx_offset, void *scratch, int device, cudaStream_t s, const PeerXchg *px = nullptr,
                          LaunchChain *chain = nullptr, float *spare_v = nullptr);
// Kernels with bounded device-side waits report an expired wait in a host-visible word, one per
// device; this returns and clears it (0 = nothing happened).
int take_reduce_status(int device);
// The cross-GPU step for a vector result: every rank's `partial[0..m)` summed in rank order into
// `out[0..m)` on every rank (m at most peer_vector_max()); see peer_vector_sum_kernel.
// Most blocks a sum in unsplit order may have (the window's block area holds that many words per generation).
uint64_t peer_blocks_max();
cudaError_t launch_peer_vector_sum(const PeerXchg &px, const float *partial, uint64_t m, float *out, int device, cudaStream_t s);
uint64_t peer_vector_max();
// Per column of [g, m] candidates (value, position), the position of the best one.
cudaError_t launch_argmax_combine(const float *vals, const int64_t *idx, uint64_t g, uint64_t m, int64_t *out, cudaStream_t s);

}  // namespace b200

// Counts and checks one kernel launch.
#define B200_LAUNCH(kernel, grid, block, smem, stream, ...)                         \
    do {                                                                            \
        kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);                 \
        ::b200::g_kernel_launches.fetch_add(1, std::memory_order_relaxed);          \
    } while (0)

// Every kernel of this library that is not one of the chained reductions starts with ordered_start():
// it may be SCHEDULED while the kernel before it in the stream is still draining (launch latency, CTA
// set-up and parameter loads overlap that kernel's tail), but it touches no memory before that kernel
// has completed and its writes are visible, so results and their order are those of plain stream
// order. It then lets the kernel after it be scheduled the same way. Launched the ordinary way, both
// instructions return at once.
namespace b200 {
__device__ __forceinline__ void ordered_start() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Whether kernels are launched for early scheduling at all (PYTORCHES_B200_OVERLAP=0 turns it off).
bool overlap_enabled();
}  // namespace b200

// Launch of a kernel that begins with ordered_start().
#define B200_LAUNCH_ORDERED(kernel, grid, block, smem, stream, ...) \
    B200_LAUNCH_OVERLAP(::b200::overlap_enabled(), kernel, grid, block, smem, stream, __VA_ARGS__)

// The same, optionally with programmatic stream serialization: the kernel may start once every CTA of
// the kernel before it in the stream has signalled (griddepcontrol.launch_dependents) or exited,
// instead of after that kernel has completed. Only for kernels written for it (see LaunchChain).
#define B200_LAUNCH_OVERLAP(overlap, kernel, grid_, block_, smem_, stream_, ...)                          \
    do {                                                                                              \
        cudaLaunchConfig_t cfg_ = {};                                                                 \
        cfg_.gridDim = dim3(grid_);                                                                   \
        cfg_.blockDim = dim3(block_);                                                                  \
        cfg_.dynamicSmemBytes = (smem_);                                                              \
        cfg_.stream = (stream_);                                                                     \
        cudaLaunchAttribute attr_[1];                                                                 \
        attr_[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                             \
        attr_[0].val.programmaticStreamSerializationAllowed = 1;                                      \
        cfg_.attrs = attr_;                                                                           \
        cfg_.numAttrs = (overlap) ? 1 : 0;                                                            \
        (void)cudaLaunchKernelEx(&cfg_, kernel, __VA_ARGS__);                                         \
        ::b200::g_kernel_launches.fetch_add(1, std::memory_order_relaxed);                            \
    } while (0)
