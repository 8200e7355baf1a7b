// Reduction kernels of the B200 plugin: SUM_AXIS (in place of plugins/cpu/src/reduce.rs) and the
// appended MAX_AXIS / ARGMAX_AXIS, over the middle axis of a contiguous (outer, len, inner) tensor.
//
// SUM reproduces the reference's association order, so its results carry the reference's bits:
//   * inner == 1 (reduce.rs:110-131): a row is cut into 65536-element blocks. Within a block element i
//     is accumulated, in order, into slot i mod 32; the 32 slots are combined pairwise at distances
//     8, 16, 4, 2, 1; the last (block length mod 32) elements are then added one by one; block sums
//     are added in block order starting from 0.0. A warp is exactly that machine: lane j owns slot j
//     (its loads, x[32k + j], are perfectly coalesced), and the slot combine is a shuffle tree with
//     the same distances. Pass 1 gives one warp to every (row, block); pass 2, only needed when a row
//     has more than one block, adds a row's block sums in order. No atomics, so reruns are identical.
//   * inner > 1 (reduce.rs:132-145): every output column adds its len inputs in order from 0.0; one
//     thread per column, loads of neighbouring threads coalesce.
// MAX / ARGMAX have no reference implementation; they follow torch CPU (NaN wins, first index on
// ties). max is order-independent, so these use float4 loads and a two-pass (value, index) combine.
//
// All kernels are pure HBM streaming: every load of a thread's batch is issued before the first use.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include <cuda.h>  // CUtensorMap and its enums only; the encoder is looked up at run time, libcuda is not linked

#include "common.cuh"

namespace b200 {

namespace {

constexpr uint64_t SUM_BLOCK = 1ull << 16;  // reduce.rs:10
constexpr int SUM_WARPS = 2;                // warps per CTA in pass 1
constexpr int SUM_UNROLL = 16;              // loads in flight per lane

__device__ __forceinline__ float ldf(const float *p) { return __ldcs(p); }
__device__ __forceinline__ float4 ldf4(const float *p) { return __ldcs(reinterpret_cast<const float4 *>(p)); }

// Sum of m <= 65536 contiguous elements in the reference's order (reduce.rs:36-61). Whole warp calls;
// the result is valid in lane 0.
__device__ __forceinline__ float warp_block_sum(const float *__restrict__ p, uint32_t m, int lane) {
    const uint32_t m32 = m & ~31u;
    float s = 0.0f;
    uint32_t k = lane;
    for (; k + 32 * (SUM_UNROLL - 1) < m32; k += 32 * SUM_UNROLL) {
        float v[SUM_UNROLL];
#pragma unroll
        for (int u = 0; u < SUM_UNROLL; ++u) v[u] = ldf(p + k + 32 * u);
#pragma unroll
        for (int u = 0; u < SUM_UNROLL; ++u) s = __fadd_rn(s, v[u]);
    }
    for (; k < m32; k += 32) s = __fadd_rn(s, ldf(p + k));
    // (a0+a1)+(a2+a3), then high half onto low half, then lanes (0+2),(1+3), then those two.
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 8));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 16));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 4));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 2));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 1));
    if (lane == 0)
        for (uint32_t i = m32; i < m; ++i) s = __fadd_rn(s, p[i]);
    return s;
}

// Pass 1, inner == 1: warp t handles block (t mod blocks) of row (t div blocks). With one block per
// row the row's result is written directly as 0.0 + block sum (the reference's combine loop).
__global__ void __launch_bounds__(32 * SUM_WARPS) sum_rows_kernel(const float *__restrict__ x, uint64_t tasks, uint64_t len,
                                                                  uint64_t blocks, float *__restrict__ dst) {
    ordered_start();
    const uint64_t t = (uint64_t)blockIdx.x * SUM_WARPS + (threadIdx.x >> 5);
    if (t >= tasks) return;
    const int lane = threadIdx.x & 31;
    const uint64_t row = t / blocks, b = t - row * blocks;
    const uint64_t lo = b * SUM_BLOCK;
    const uint32_t m = (uint32_t)(len - lo < SUM_BLOCK ? len - lo : SUM_BLOCK);
    const float s = warp_block_sum(x + row * len + lo, m, lane);
    if (lane == 0) dst[t] = blocks == 1 ? __fadd_rn(0.0f, s) : s;
}

// ---- pass 1 for long rows: TMA-staged -------------------------------------------------------------------
// The order constraint fixes the parallelism at one warp per 65536 elements, too few warps to keep
// HBM busy with register loads. So the warp lets the TMA engine do the loading: lane 0 keeps
// STAGES bulk copies of CHUNK floats (16 KiB each in the usual shapes) in flight into a
// shared-memory ring, each completing on an mbarrier; the warp then reads a landed chunk at stride 32
// (lane j takes words j, j+32, ...: conflict-free, and exactly "element i goes to slot i mod 32") and
// adds in order. One warp per CTA; shared memory decides how many CTAs an SM holds.
// Bulk copies need 16-byte aligned sources; the host picks this kernel only when every block start is.
//
// Every wait is bounded. If a barrier does not complete within the limit the warp gives its other
// copies in flight the same bounded chance to land, records WAIT_EXPIRED in *status (pinned host
// memory the next blocking call inspects) and returns without a result.
//
// The ring's shape is a template parameter, picked from the grid (see pick_ring): a long row has
// thousands of blocks, CTAs come and go in many waves and a deep ring (4 x 16 KiB, three CTAs per SM)
// keeps HBM busy; a row of a few hundred blocks (a 128 MiB shard has 512) fits the GPU all at once
// if the ring is shallow (2 x 16 KiB, six CTAs per SM), and then nothing waits for a second wave.
constexpr uint32_t TMA_MIN_CHUNK = 4096;  // floats; rows shorter than 8 of these take the register-load kernel
constexpr size_t ring_bytes(int stages, uint32_t chunk) { return (size_t)stages * chunk * 4; }
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // try_wait calls before giving up (each may block briefly)
constexpr int STATUS_WAIT_EXPIRED = 1;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (uint32_t tries = 0; tries < WAIT_LIMIT; ++tries)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Bulk copy from global memory into this CTA's own shared memory. `policy` (read_once_policy): the
// data is read once, so L2 may drop it first. A reduction streams its whole input through L2; left at
// normal priority that pushes out the few lines everything else waits on (the combiners' mailbox and
// window words), and a combiner that has to fetch them from DRAM again queues behind megabytes of
// bulk copies in flight: several microseconds per look.
__device__ __forceinline__ uint64_t read_once_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
                 : "memory");
}

// Programmatic dependent launch. launch_dependents: "as far as this CTA is concerned, the next kernel
// in the stream may start"; it starts once every CTA of this grid has said so or exited.
// wait_for_prior_grid: blocks until the kernel before this one in the stream has completed and its
// writes are visible (returns at once if this kernel was launched the ordinary way).
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

constexpr uint32_t POLL_LIMIT = 1u << 21;  // polls of a mailbox word (or of `done`) before giving up

// How the combiner CTAs of back-to-back reductions keep order while up to THREE of these kernels are
// in flight. `done` is a per-device word holding the launch number (`epoch`, consecutive per device)
// of the newest such kernel that has finished. A combiner
//   * begins by waiting (bounded) until the kernel two before its own has finished, and only then
//     lets the kernel after its own start: kernels e-1, e and e+1 may overlap, e+2 may not start
//     before e-1 is done, so four mailbox regions and eight window generations used in turn never
//     collide (a rank cannot finish a reduction without every peer's part, which bounds the skew);
//   * works (polls, chains, exchanges) at once, whatever the kernels before it are doing: the chain of
//     a sum in unsplit order, 4096 dependent adds, thus has two kernels' streaming to hide behind;
//   * ends by waiting for the kernel before its own to complete (griddepcontrol.wait) and then
//     publishing its number: completion is in launch order, so whatever is launched the ordinary way
//     after these kernels, waiting for the last, waits for all of them.
// A wait that runs out is reported through *status like every other bounded wait; the combiner still
// lets its dependents start and still publishes its number, so one failure does not stall the stream.
__device__ __forceinline__ void combiner_begin(unsigned long long *done, uint32_t epoch, int *status, uint32_t lag) {
    bool ok = false;
    for (uint32_t tries = 0; tries < POLL_LIMIT; ++tries) {
        unsigned long long d;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(d) : "l"(done) : "memory");
        if ((long long)(d + lag - (unsigned long long)epoch) >= 0) {
            ok = true;
            break;
        }
    }
    if (!ok && (threadIdx.x & 31) == 0) {
        *(volatile int *)status = STATUS_WAIT_EXPIRED;
        __threadfence_system();
    }
    launch_dependents();
}
// One thread of the combiner CTA calls this after everything else the CTA does.
__device__ __forceinline__ void combiner_end(unsigned long long *done, uint32_t epoch) {
    wait_for_prior_grid();
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(done), "l"((unsigned long long)epoch) : "memory");
}

// FUSED (one row only): the ordered chain over the block sums runs INSIDE this launch. CTA 0 is the
// combiner; CTAs 1..blocks are the workers. A worker publishes its block sum as ONE 64-bit word,
// (epoch << 32) | float bits, into a per-device mailbox; the combiner polls the words in block order
// (the mailbox persists between launches and every launch has a new epoch, so a word of this launch
// cannot be mistaken for an old one and nothing needs clearing), adds each sum as soon as it is there
// and writes the result. With 4096 workers taking three CTA slots per SM at a time, block sums arrive
// in waves and the chain hides behind the streaming; only the last wave's sums are added after it.
// A 64-bit aligned store is indivisible, so no fence and no atomic is needed, and the order of the
// adds (hence the bits) is the reference's. The combiner's polls are bounded like every other wait.

__device__ __forceinline__ unsigned long long ld_mailbox(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}


__device__ __forceinline__ bool vi_better(float v, uint64_t i, float bv, uint64_t bi);

// ---- the cross-GPU step --------------------------------------------------------------------------------------
// Called by one whole warp with the same (v, pos) in every lane: this GPU's result. Lane r < world
// stores it into slot `rank` of rank r's window (its own window included) and then waits for slot r
// of its OWN window to be filled by rank r. A slot is two 64-bit words: the position, written first,
// then (epoch << 32) | float bits, written with release semantics at system scope; the reader polls
// that word with acquire loads until it carries this reduction's epoch. Eight generations of slots are
// used in turn, so a fast rank's later reduction never lands on a slot a slow rank has yet to read: a
// rank starts reduction s only after its own combiner of s-3 has finished (see combiner_begin), which
// needed every peer's part of s-3, and a peer working on s-3 has finished reading everything up to s-6.
// The wait is bounded in time; if a peer never shows up the warp records it in *status and returns
// false without a result, and the host reports the failure at its next blocking call.
constexpr int PEER_GENERATIONS = 8;
constexpr int PEER_SLOT_WORDS = 2;
constexpr size_t PEER_WINDOW_WORDS = (size_t)PEER_GENERATIONS * PEER_MAX_RANKS * PEER_SLOT_WORDS;
constexpr int STATUS_PEER_WAIT_EXPIRED = 2;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void peer_trace(const PeerXchg &px, int what);  // leaves a %globaltimer reading in this rank's window (below)

__device__ __forceinline__ bool peer_allgather(const PeerXchg &px, float v, int64_t pos, float &rv, int64_t &rp, int *status) {
    const int lane = threadIdx.x & 31;
    const size_t gen = (size_t)(px.epoch % PEER_GENERATIONS) * PEER_MAX_RANKS * PEER_SLOT_WORDS;
    bool ok = true;
    rv = 0.0f;
    rp = 0;
    // The window table sits in the kernel's parameter space: picked with compares, not indexed, so that it stays there.
    unsigned long long *to = px.window[0], *mine = px.window[0];
#pragma unroll
    for (int r = 1; r < PEER_MAX_RANKS; ++r) {
        if (lane == r) to = px.window[r];
        if (px.rank == r) mine = px.window[r];
    }
    if (lane < px.world) {
        unsigned long long *dst = to + gen + (size_t)px.rank * PEER_SLOT_WORDS;
        const unsigned long long w = ((unsigned long long)px.epoch << 32) | __float_as_uint(v);
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + 1), "l"((unsigned long long)pos) : "memory");
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
        const unsigned long long *src = mine + gen + (size_t)lane * PEER_SLOT_WORDS;
        const unsigned long long t0 = global_ns(), limit = (unsigned long long)px.wait_ms * 1000000ull;
        ok = false;
        for (uint32_t tries = 0; tries < (1u << 30); ++tries) {  // the time limit ends the loop; the count is a second guard
            unsigned long long got;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
            if ((uint32_t)(got >> 32) == px.epoch) {
                unsigned long long p2;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(p2) : "l"(src + 1) : "memory");
                rv = __uint_as_float((uint32_t)got);
                rp = (int64_t)p2;
                ok = true;
                break;
            }
            if ((tries & 63) == 63 && global_ns() - t0 > limit) break;
        }
    }
    if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) {
            *(volatile int *)status = STATUS_PEER_WAIT_EXPIRED;
            __threadfence_system();
        }
        return false;
    }
    return true;
}

// Exchanges this GPU's result with the peers and combines all of them in rank order, exactly as the
// same plugin op would combine a [world] tensor of the per-rank results: SUM adds them one by one to
// 0.0 and adds that to 0.0 (the row path for rows shorter than 32, sum_short_rows_kernel), and then
// divides by px.divide_by if that is set (a mean); MAX and
// MAX_ARGMAX keep the best (value, position): NaN wins, then the larger value, then the lower position.
// Whole warp, same (v, pos) in every lane; lane 0 writes. Returns without writing if the wait expired.
__device__ __forceinline__ void peer_finish(const PeerXchg &px, int kind, float v, int64_t pos, float *out_v, int64_t *out_i, int *status) {
    const int lane = threadIdx.x & 31;
    float rv;
    int64_t rp;
    if (lane == 0) peer_trace(px, 1);
    if (!peer_allgather(px, v, pos, rv, rp, status)) return;
    if (lane == 0) peer_trace(px, 2);
    if (kind == REDUCE_SUM) {
        float s = 0.0f;
        for (int r = 0; r < px.world; ++r) s = __fadd_rn(s, __shfl_sync(0xffffffffu, rv, r));
        s = __fadd_rn(0.0f, s);
        // A mean is the reference's sum followed by a DIV by the element count as an f32 scalar
        // (crates/core/src/lib.rs:662-670): one IEEE division, the same bits as FILL + DIV.
        if (px.divide_by != 0.0f) s = __fdiv_rn(s, px.divide_by);
        if (lane == 0) {
            out_v[0] = s;
            peer_trace(px, 3);
        }
        return;
    }
    float bv = lane < px.world ? rv : __int_as_float(0xff800000);
    uint64_t bp = lane < px.world ? (uint64_t)rp : ~0ull;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
        const uint64_t op = __shfl_xor_sync(0xffffffffu, bp, d);
        if (vi_better(ov, op, bv, bp)) { bv = ov; bp = op; }
    }
    if (lane == 0) {
        if (out_v) out_v[0] = bv;
        if (out_i) out_i[0] = (int64_t)bp;
        peer_trace(px, 3);
    }
}

// The cross-GPU step alone, for reductions whose local part did not end in a combiner CTA (short
// inputs): reads this GPU's finished result from the output locations and overwrites them.
__global__ void __launch_bounds__(32) peer_exchange_kernel(const __grid_constant__ PeerXchg px, int kind, float *v, int64_t *i, int *status) {
    ordered_start();
    peer_finish(px, kind, v ? v[0] : 0.0f, i ? i[0] : (int64_t)px.rank, v, i, status);  // no position: the rank breaks ties
}

// ---- the cross-GPU step for small VECTOR results (a bias gradient: the sum over a sharded leading
// dimension of a [rows, m] tensor, m up to PEER_VECTOR_MAX) ---------------------------------------------
// The same idea as above, one word per element: thread j stores (epoch << 32) | bits(partial[j]) into
// element j of slot `rank` of EVERY rank's window (plain peer stores; each 64-bit word validates
// itself, so no ordering between words is needed), then polls element j of every rank's slot in its
// OWN window until it carries this epoch, and adds the values in rank order from 0.0: what SUM_AXIS
// over the gathered [world, m] tensor computes (reduce.rs:132-145), on every rank alike. The vector
// area of a window follows its scalar area: PEER_GENERATIONS x PEER_MAX_RANKS slots of
// PEER_VECTOR_MAX words, generations used in turn exactly as for scalars. Waits are bounded in time.
constexpr uint32_t PEER_VECTOR_MAX = 4096;           // elements (16 KiB of f32)
constexpr size_t PEER_VECTOR_AREA_WORD = 512;        // first word of the vector area (the scalar area ends before it)
// After the vector area: the block area for sums in unsplit order, PEER_GENERATIONS x PEER_BLOCKS_MAX
// words, one per 65536-element block of the whole tensor (2^30 elements at most).
constexpr uint32_t PEER_BLOCKS_MAX = 16384;
constexpr size_t PEER_BLOCK_AREA_WORD = PEER_VECTOR_AREA_WORD + (size_t)PEER_GENERATIONS * PEER_MAX_RANKS * PEER_VECTOR_MAX;
// Beside the window, in ordinary memory of the device: a trace of its last PEER_TRACE_RECORDS reductions,
// PEER_TRACE_WORDS words each (record = epoch mod PEER_TRACE_RECORDS), %globaltimer readings: [1] this
// GPU's own part is complete (its result ready to send, or its last block sum forwarded), [2] every
// rank's part has arrived here, [3] the result is written; a sum in unsplit order adds [13], the
// number of bulk copies its combiner needed (a count); the rest is unused. [2] - [1] is the wait for the slowest
// peer (skew plus NVLink latency; in unsplit order it also holds this combiner's wait for the kernel
// before it), [3] - [2] what is left to do after the last arrival. Read back with
// pytorches_b200_peer_trace. (A reading at the combiner's start was dropped: a store placed right
// behind griddepcontrol.launch_dependents, even one that never executes, cost 12% of the step at 2
// GPUs and 40% at 4 with sums in unsplit order.)
constexpr uint32_t PEER_TRACE_RECORDS = 64;
constexpr uint32_t PEER_TRACE_WORDS = 16;

__device__ __forceinline__ unsigned long long *own_window(const PeerXchg &px) {
    unsigned long long *mine = px.window[0];
#pragma unroll
    for (int r = 1; r < PEER_MAX_RANKS; ++r)
        if (px.rank == r) mine = px.window[r];
    return mine;
}
__device__ __forceinline__ void peer_trace(const PeerXchg &px, int what) {
    if (px.trace) px.trace[(size_t)(px.epoch % PEER_TRACE_RECORDS) * PEER_TRACE_WORDS + what] = global_ns();
}

__global__ void __launch_bounds__(256) peer_vector_sum_kernel(const __grid_constant__ PeerXchg px, const float *__restrict__ partial, uint32_t m,
                                                              float *__restrict__ out, int *status) {
    ordered_start();
    const uint32_t j = blockIdx.x * 256 + threadIdx.x;
    bool ok = true;
    if (j < m) {
        const size_t gen = PEER_VECTOR_AREA_WORD + (size_t)(px.epoch % PEER_GENERATIONS) * PEER_MAX_RANKS * PEER_VECTOR_MAX;
        const unsigned long long w = ((unsigned long long)px.epoch << 32) | __float_as_uint(partial[j]);
        unsigned long long *mine = px.window[0];
#pragma unroll
        for (int r = 0; r < PEER_MAX_RANKS; ++r) {
            if (r < px.world) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(px.window[r] + gen + (size_t)px.rank * PEER_VECTOR_MAX + j), "l"(w) : "memory");
            if (px.rank == r) mine = px.window[r];
        }
        const unsigned long long t0 = global_ns(), limit = (unsigned long long)px.wait_ms * 1000000ull;
        float s = 0.0f;
        for (int r = 0; r < px.world && ok; ++r) {
            const unsigned long long *src = mine + gen + (size_t)r * PEER_VECTOR_MAX + j;
            ok = false;
            for (uint32_t tries = 0; tries < (1u << 30); ++tries) {  // the time limit ends the loop; the count is a second guard
                unsigned long long got;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
                if ((uint32_t)(got >> 32) == px.epoch) {
                    s = __fadd_rn(s, __uint_as_float((uint32_t)got));
                    ok = true;
                    break;
                }
                if ((tries & 63) == 63 && global_ns() - t0 > limit) break;
            }
        }
        if (ok) out[j] = s;
    }
    if (!ok) {
        *(volatile int *)status = STATUS_PEER_WAIT_EXPIRED;
        __threadfence_system();
    }
}

// A poll is a round trip to L2 (a microsecond or more under load), so the combiner fetches 512 words
// per round (16 per lane, all in flight together), issues the NEXT round's loads before it chains the
// current round's 512 dependent adds (about a microsecond, so the round trip hides behind the chain
// once the words are there), and re-polls only the words not yet published.
constexpr int COMBINER_WORDS = 16;

// s + f[0] + f[1] + ... + f[n-1], in that order, out of shared memory: every lane runs the same chain
// with 16-byte broadcast loads, four sums per load, the next loads in flight while the current four
// adds run, so the chain advances at the add latency. `f` is 16-byte aligned; up to 16 floats past
// f[n-1] are read and dropped, so they must lie inside the CTA's shared memory.
__device__ __forceinline__ float chain_staged(const float *f, uint32_t n, float s) {
    const float4 *quad = reinterpret_cast<const float4 *>(f);
    float4 cur[4], nxt[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) cur[u] = quad[u];
    uint32_t i = 0;
    for (; i + 32 <= n; i += 32) {  // 32 sums per trip: two batches of four float4
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            nxt[u] = quad[i / 4 + 4 + u];
            s = __fadd_rn(s, cur[u].x);
            s = __fadd_rn(s, cur[u].y);
            s = __fadd_rn(s, cur[u].z);
            s = __fadd_rn(s, cur[u].w);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            cur[u] = quad[i / 4 + 8 + u];
            s = __fadd_rn(s, nxt[u].x);
            s = __fadd_rn(s, nxt[u].y);
            s = __fadd_rn(s, nxt[u].z);
            s = __fadd_rn(s, nxt[u].w);
        }
    }
    for (; i < n; ++i) s = __fadd_rn(s, f[i]);
    return s;
}

__device__ void ordered_combiner_body(const unsigned long long *mailbox, uint32_t epoch, uint64_t blocks, float *out, int *status,
                                      const PeerXchg &px, float *stage) {
    const int lane = threadIdx.x;
    float s = 0.0f;
    constexpr uint64_t ROUND = 32 * COMBINER_WORDS;
    unsigned long long w[COMBINER_WORDS];  // the round whose loads are in flight
    auto issue = [&](uint64_t base) {
#pragma unroll
        for (int k = 0; k < COMBINER_WORDS; ++k)
            if (base + k * 32 + lane < blocks) w[k] = ld_mailbox(mailbox + base + k * 32 + lane);
    };
    issue(0);
    for (uint64_t base = 0; base < blocks; base += ROUND) {
        float v[COMBINER_WORDS];
        uint32_t missing = 0;
#pragma unroll
        for (int k = 0; k < COMBINER_WORDS; ++k) {  // what the loads issued a round ago brought
            v[k] = 0.0f;
            if (base + k * 32 + lane < blocks) {
                if ((uint32_t)(w[k] >> 32) == epoch) v[k] = __uint_as_float((uint32_t)w[k]);
                else missing |= 1u << k;
            }
        }
        for (uint32_t tries = 0; tries < POLL_LIMIT && __any_sync(0xffffffffu, missing != 0); ++tries) {
            unsigned long long again[COMBINER_WORDS];
#pragma unroll
            for (int k = 0; k < COMBINER_WORDS; ++k)
                if (missing & (1u << k)) again[k] = ld_mailbox(mailbox + base + k * 32 + lane);
#pragma unroll
            for (int k = 0; k < COMBINER_WORDS; ++k)
                if ((missing & (1u << k)) && (uint32_t)(again[k] >> 32) == epoch) {
                    v[k] = __uint_as_float((uint32_t)again[k]);
                    missing &= ~(1u << k);
                }
        }
        if (__any_sync(0xffffffffu, missing != 0)) {
            if (lane == 0) {
                *(volatile int *)status = STATUS_WAIT_EXPIRED;
                __threadfence_system();
            }
            return;
        }
        if (base + ROUND < blocks) issue(base + ROUND);  // in flight while this round is chained
        // The round's sums go through shared memory (this CTA's ring is otherwise unused) so that every
        // lane can run the same chain with 16-byte broadcast loads, four sums per load, the next loads
        // in flight while the current four adds run: the chain advances at the add latency. (Fetching
        // each sum from its lane with a shuffle costs five times that.)
        __syncwarp();
#pragma unroll
        for (int k = 0; k < COMBINER_WORDS; ++k) stage[k * 32 + lane] = v[k];
        __syncwarp();
        const uint32_t count = (uint32_t)(blocks - base < ROUND ? blocks - base : ROUND);
        s = chain_staged(stage, count, s);
    }
    if (px.world > 0) return peer_finish(px, REDUCE_SUM, s, 0, out, nullptr, status);  // s is the same in every lane
    if (lane == 0) out[0] = s;
}

// The combiner of a sum in unsplit order. `words` = this reduction's generation of the block area of
// this rank's own window, one (epoch << 32 | bits) word per block of the WHOLE tensor, written by
// every rank's forwarder. The chain over them is serial and must follow block order, and on G GPUs
// all but the first GPU's last blocks are there long before their turn: when the last block sums
// arrive, about (G-1)/G of the chain is still to run. What must not be paid then is a memory round
// trip per few hundred words: under the streaming of the kernels that follow, a load that misses L2
// queues behind megabytes of bulk copies, microseconds each time. So the words are fetched the way
// the workers fetch their input: ONE bulk copy brings every word from the chain's position on (up to
// UNSPLIT_WINDOW of them, 32 KiB) into shared memory; the warp finds how far the words of this
// reduction reach without a gap, asks for the next copy into the other buffer, and chains what it
// has out of shared memory meanwhile. After the last arrival that is at most two copies and one pass
// of the chain. A word is written by one aligned 8-byte store and a bulk copy moves aligned 16-byte
// units, so a word is seen whole or not at all; a copy that overtakes a store only costs another
// round. Waits are bounded: each copy by the barrier's try limit, the whole by px.wait_ms.
constexpr uint32_t UNSPLIT_WINDOW = 4096;                                  // words per copy
constexpr size_t UNSPLIT_SMEM = (size_t)2 * UNSPLIT_WINDOW * 8;            // two buffers
// Dynamic shared memory of a fused launch: the workers' ring, and room for the unsplit combiner's buffers
// (every CTA of a launch gets the same; 64 KiB still lets three CTAs share an SM).
constexpr size_t fused_smem(int stages, uint32_t chunk, bool unsplit) {
    return unsplit && ring_bytes(stages, chunk) < UNSPLIT_SMEM ? UNSPLIT_SMEM : ring_bytes(stages, chunk);
}
__device__ void unsplit_combiner(const unsigned long long *words, uint32_t epoch, uint64_t blocks, float *out, int *status, const PeerXchg &px,
                                 unsigned char *smem, uint64_t *bars) {
    const int lane = threadIdx.x;
    if (lane == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const unsigned long long t0 = global_ns(), limit = (unsigned long long)px.wait_ms * 1000000ull;
    // Copy number f lands in buffer f & 1 on bars[f & 1], whose phase it completes is (f >> 1) & 1.
    auto fetch = [&](uint32_t f, uint64_t from, uint64_t &first, uint32_t &count) {  // one lane asks
        first = from & ~1ull;  // 16-byte aligned
        const uint64_t left = blocks - first;
        count = (uint32_t)(left < UNSPLIT_WINDOW ? (left + 1) & ~1ull : UNSPLIT_WINDOW);  // a whole number of 16 bytes (the area has room)
        if (lane == 0) {
            // Generic-proxy reads of this buffer (the chain before) are ordered before the async-proxy write.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&bars[f & 1], count * 8);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             smem_addr(smem + (size_t)(f & 1) * UNSPLIT_WINDOW * 8)),
                         "l"(words + first), "r"(count * 8), "r"(smem_addr(&bars[f & 1]))
                         : "memory");
        }
    };
    float s = 0.0f;
    uint64_t pos = 0;            // next block to add
    uint64_t base = 0, base_next = 0;  // first word the landed / the requested copy holds
    uint32_t held = 0, held_next = 0;  // how many
    bool failed = false;
    uint32_t f = 0;              // the copy being waited for
    fetch(0, 0, base, held);
    while (true) {
        if (!mbar_wait_bounded(&bars[f & 1], (f >> 1) & 1)) {
            failed = true;
            break;
        }
        // How far do this reduction's words reach from `pos`? Each lane looks at every 32nd word and, on
        // the way, packs the low halves (the sums) to the front of the same buffer: word i of the
        // buffer becomes float i. Four steps of 32 words are read before they are written; a step's
        // floats land on words that earlier steps have read.
        unsigned long long *wbuf = reinterpret_cast<unsigned long long *>(smem + (size_t)(f & 1) * UNSPLIT_WINDOW * 8);
        float *fbuf = reinterpret_cast<float *>(wbuf);
        const uint32_t k0 = (uint32_t)(pos - base), k_end = (uint32_t)(blocks - base < held ? blocks - base : held);
        uint32_t first_gap = k_end;
        for (uint32_t k = k0 & ~127u; k < k_end; k += 128) {
            unsigned long long w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = k + u * 32 + lane < held ? wbuf[k + u * 32 + lane] : 0ull;
            __syncwarp();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = k + u * 32 + lane;
                if (i < held) fbuf[i] = __uint_as_float((uint32_t)w[u]);
                if (i >= k0 && i < k_end && (uint32_t)(w[u] >> 32) != epoch && i < first_gap) first_gap = i;
            }
            __syncwarp();
        }
        first_gap = __reduce_min_sync(0xffffffffu, first_gap);
        const uint64_t reach = base + first_gap;
        const bool complete = reach == blocks;
        if (complete && lane == 0) peer_trace(px, 2);  // every rank's part has arrived
        if (!complete) {
            if (__any_sync(0xffffffffu, global_ns() - t0 > limit)) {
                failed = true;
                break;
            }
            fetch(f + 1, reach, base_next, held_next);  // in flight while the chain below runs
        }
        // chain floats k0 .. first_gap: singly up to a 16-byte boundary, then staged
        uint32_t k = k0;
        for (; k < first_gap && (k & 3) != 0; ++k) s = __fadd_rn(s, fbuf[k]);
        if (k < first_gap) s = chain_staged(fbuf + k, first_gap - k, s);
        pos = reach;
        if (complete) break;
        ++f;
        base = base_next;
        held = held_next;
    }
    if (failed) {
        // Nothing is on its way into shared memory here: either the one copy in flight had its bounded
        // chance and never landed, or time ran out between two copies.
        if (lane == 0) {
            *(volatile int *)status = STATUS_PEER_WAIT_EXPIRED;
            __threadfence_system();
        }
        return;
    }
    if (px.divide_by != 0.0f) s = __fdiv_rn(s, px.divide_by);
    if (lane == 0) {
        out[0] = s;
        peer_trace(px, 3);
        if (px.trace) px.trace[(size_t)(px.epoch % PEER_TRACE_RECORDS) * PEER_TRACE_WORDS + 13] = f + 1;
    }
}

// `launch_no`: this kernel's number among the device's chained reductions (see combiner_begin).
__device__ void ordered_combiner(const unsigned long long *mailbox, uint32_t epoch, uint64_t blocks, float *out, int *status,
                                 const PeerXchg &px, float *stage, unsigned long long *done, uint32_t launch_no, uint32_t lag, uint64_t *bars) {
    combiner_begin(done, launch_no, status, lag);
    if (px.blocks_total != 0) unsplit_combiner(mailbox, epoch, blocks, out, status, px, reinterpret_cast<unsigned char *>(stage), bars);
    else ordered_combiner_body(mailbox, epoch, blocks, out, status, px, stage);
    __syncwarp();
    if (threadIdx.x == 0) combiner_end(done, launch_no);
}

// Unsplit order, second special CTA: hands this GPU's block sums to every rank. The workers publish
// into the local mailbox exactly as they do on one GPU (a store across NVLink at the end of a worker
// would keep its SM slot busy for the round trip, 1024 times per reduction); this warp polls the local
// words in rounds and, as they appear, stores each as (group epoch << 32) | bits into the block area of
// EVERY rank's window, its own included, from where the combiners chain them.
__device__ void block_forwarder(const unsigned long long *mailbox, uint32_t epoch, uint64_t blocks, int *status, const PeerXchg &px) {
    const int lane = threadIdx.x;
    const size_t at = PEER_BLOCK_AREA_WORD + (size_t)(px.epoch % PEER_GENERATIONS) * PEER_BLOCKS_MAX + px.block0;
    for (uint64_t base = 0; base < blocks; base += 32 * COMBINER_WORDS) {
        uint32_t missing = 0;
#pragma unroll
        for (int k = 0; k < COMBINER_WORDS; ++k)
            if (base + k * 32 + lane < blocks) missing |= 1u << k;
        for (uint32_t tries = 0; tries < POLL_LIMIT && __any_sync(0xffffffffu, missing != 0); ++tries) {
            unsigned long long w[COMBINER_WORDS];
#pragma unroll
            for (int k = 0; k < COMBINER_WORDS; ++k)
                if (missing & (1u << k)) w[k] = ld_mailbox(mailbox + base + k * 32 + lane);
#pragma unroll
            for (int k = 0; k < COMBINER_WORDS; ++k)
                if ((missing & (1u << k)) && (uint32_t)(w[k] >> 32) == epoch) {
                    missing &= ~(1u << k);
                    const unsigned long long out = ((unsigned long long)px.epoch << 32) | (uint32_t)w[k];
#pragma unroll
                    for (int r = 0; r < PEER_MAX_RANKS; ++r)
                        if (r < px.world) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(px.window[r] + at + base + k * 32 + lane), "l"(out) : "memory");
                }
        }
        if (__any_sync(0xffffffffu, missing != 0)) {
            if (lane == 0) {
                *(volatile int *)status = STATUS_WAIT_EXPIRED;
                __threadfence_system();
            }
            return;
        }
    }
    if (lane == 0) peer_trace(px, 1);
}

template <bool FUSED, int STAGES, uint32_t CHUNK>
__global__ void __launch_bounds__(32) sum_rows_tma_kernel(const float *__restrict__ x, uint64_t tasks, uint64_t len, uint64_t blocks,
                                                          float *__restrict__ dst, int *status, unsigned long long *mailbox, uint32_t epoch,
                                                          const __grid_constant__ PeerXchg px, uint32_t ordered, unsigned long long *done) {
    constexpr uint32_t CHUNK_BYTES = CHUNK * 4;
    extern __shared__ __align__(128) unsigned char tma_smem[];
    __shared__ uint64_t bars[STAGES];
    float *ring = reinterpret_cast<float *>(tma_smem);
    if (FUSED && blockIdx.x == 0) {
        if (px.blocks_total != 0) {  // unsplit order: chain the whole tensor's block sums out of this rank's own window
            const unsigned long long *mine = own_window(px);
            return ordered_combiner(mine + PEER_BLOCK_AREA_WORD + (size_t)(px.epoch % PEER_GENERATIONS) * PEER_BLOCKS_MAX, px.epoch, px.blocks_total, dst,
                                    status, px, ring, done, epoch, ordered >> 8, bars);
        }
        return ordered_combiner(mailbox, epoch, blocks, dst, status, px, ring, done, epoch, ordered >> 8, bars);
    }
    // `ordered`: what came before in the stream may have written this kernel's input, so it waits for
    // that to complete like every other kernel. Otherwise (the kernel before is a reduction of other
    // buffers) a worker needs nothing from it and starts streaming at once.
    if (!FUSED || (ordered & 1)) ordered_start();
    else launch_dependents();
    const bool unsplit = FUSED && px.blocks_total != 0;
    if (unsplit && blockIdx.x == 1) return block_forwarder(mailbox, epoch, blocks, status, px);
    const uint64_t t = FUSED ? blockIdx.x - (unsplit ? 2 : 1) : blockIdx.x;
    const int lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const uint64_t row = t / blocks, b = t - row * blocks;
    const uint64_t lo = b * SUM_BLOCK;
    const uint32_t m = (uint32_t)(len - lo < SUM_BLOCK ? len - lo : SUM_BLOCK);
    const float *p = x + row * len + lo;
    const uint32_t chunks = m / CHUNK;
    const uint64_t once = read_once_policy();
    if (lane == 0) {
        for (uint32_t c = 0; c < STAGES && c < chunks; ++c) {
            mbar_expect_tx(&bars[c], CHUNK_BYTES);
            bulk_load(ring + (size_t)c * CHUNK, p + (size_t)c * CHUNK, CHUNK_BYTES, &bars[c], once);
        }
    }
    float s = 0.0f;
    for (uint32_t c = 0; c < chunks; ++c) {
        const int st = c % STAGES;
        if (!mbar_wait_bounded(&bars[st], (c / STAGES) & 1)) {
            // Give the copies still in flight (chunks c+1 .. c+STAGES-1) their bounded chance, then stop.
            for (uint32_t d = c + 1; d < chunks && d < c + STAGES; ++d) (void)mbar_wait_bounded(&bars[d % STAGES], (d / STAGES) & 1);
            if (lane == 0) {
                *(volatile int *)status = STATUS_WAIT_EXPIRED;
                __threadfence_system();
            }
            return;
        }
        const float *buf = ring + (size_t)st * CHUNK;
#pragma unroll 2
        for (uint32_t k = 0; k < CHUNK / 32; k += 32) {
            float v[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) v[u] = buf[lane + 32 * (k + u)];
#pragma unroll
            for (int u = 0; u < 32; ++u) s = __fadd_rn(s, v[u]);
        }
        __syncwarp();  // every lane is done reading this stage before it is refilled
        if (lane == 0 && c + STAGES < chunks) {
            mbar_expect_tx(&bars[st], CHUNK_BYTES);
            bulk_load(ring + (size_t)st * CHUNK, p + (size_t)(c + STAGES) * CHUNK, CHUNK_BYTES, &bars[st], once);
        }
    }
    // What is left of the block (fewer than CHUNK elements) continues the same slots with loads.
    const uint32_t m32 = m & ~31u;
    for (uint32_t k = chunks * CHUNK + lane; k < m32; k += 32) s = __fadd_rn(s, ldf(p + k));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 8));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 16));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 4));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 2));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 1));
    if (lane == 0) {
        for (uint32_t i = m32; i < m; ++i) s = __fadd_rn(s, p[i]);
        if (FUSED) {
            const unsigned long long w = ((unsigned long long)epoch << 32) | __float_as_uint(s);
            asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(mailbox + t), "l"(w) : "memory");
        } else {
            dst[t] = blocks == 1 ? __fadd_rn(0.0f, s) : s;
        }
    }
}

// Rows shorter than 32 elements never fill a slot: the reference adds them one by one to 0.0.
__global__ void __launch_bounds__(256) sum_short_rows_kernel(const float *__restrict__ x, uint64_t outer, uint32_t len,
                                                             float *__restrict__ out) {
    ordered_start();
    const uint64_t r = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (r >= outer) return;
    const float *p = x + r * len;
    float s = 0.0f;
    for (uint32_t i = 0; i < len; ++i) s = __fadd_rn(s, p[i]);
    out[r] = __fadd_rn(0.0f, s);
}

// Pass 2, inner == 1: out[row] = ((0.0 + p[0]) + p[1]) + ... in block order. A CTA per row stages the
// partials through shared memory (all threads, all loads of a stage in flight at once); thread 0 runs
// the ordered chain. The chain is inherently serial, one add latency per partial, so the 32 values of
// the next step are fetched from shared memory while the current 32 are being added.
constexpr int COMBINE_THREADS = 256;
constexpr int COMBINE_STAGE = 4096;
__global__ void __launch_bounds__(COMBINE_THREADS) sum_combine_kernel(const float *__restrict__ partial, uint64_t blocks,
                                                                      float *__restrict__ out) {
    ordered_start();
    __shared__ float stage[COMBINE_STAGE + 32];
    const uint64_t row = blockIdx.x;
    const float *p = partial + row * blocks;
    float s = 0.0f;
    for (uint64_t base = 0; base < blocks; base += COMBINE_STAGE) {
        const uint32_t m = (uint32_t)(blocks - base < COMBINE_STAGE ? blocks - base : COMBINE_STAGE);
        float v[COMBINE_STAGE / COMBINE_THREADS];
#pragma unroll
        for (int u = 0; u < COMBINE_STAGE / COMBINE_THREADS; ++u) {
            const uint32_t i = threadIdx.x + COMBINE_THREADS * u;
            v[u] = i < m ? p[base + i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < COMBINE_STAGE / COMBINE_THREADS; ++u) stage[threadIdx.x + COMBINE_THREADS * u] = v[u];
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t full = m & ~31u;
            float cur[32], nxt[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) cur[u] = stage[u];
            for (uint32_t i = 0; i < full; i += 32) {
#pragma unroll
                for (int u = 0; u < 32; ++u) nxt[u] = stage[i + 32 + u];  // stage has 32 floats of slack
#pragma unroll
                for (int u = 0; u < 32; ++u) s = __fadd_rn(s, cur[u]);
#pragma unroll
                for (int u = 0; u < 32; ++u) cur[u] = nxt[u];
            }
            for (uint32_t i = full; i < m; ++i) s = __fadd_rn(s, stage[i]);
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[row] = s;
}

// inner > 1: thread per output column, rows j added in order from 0.0.
constexpr int COL_UNROLL = 8;
__global__ void __launch_bounds__(256) sum_cols_kernel(const float *__restrict__ x, uint64_t total, uint64_t len, uint64_t inner,
                                                       float *__restrict__ out) {
    ordered_start();
    const uint64_t t = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (t >= total) return;
    const uint64_t o = t / inner, i = t - o * inner;
    const float *p = x + o * len * inner + i;
    float s = 0.0f;
    uint64_t j = 0;
    for (; j + COL_UNROLL <= len; j += COL_UNROLL) {
        float v[COL_UNROLL];
#pragma unroll
        for (int u = 0; u < COL_UNROLL; ++u) v[u] = ldf(p + (j + u) * inner);
#pragma unroll
        for (int u = 0; u < COL_UNROLL; ++u) s = __fadd_rn(s, v[u]);
    }
    for (; j < len; ++j) s = __fadd_rn(s, ldf(p + j * inner));
    out[t] = s;
}

// inner > 1, TMA-staged: a one-warp CTA per group of 32 adjacent columns. Each column is still one
// ordered chain (rows 0, 1, 2, ... added to 0.0), so the parallelism is fixed at outer*inner chains and
// a chain advances one add latency per row; what can be taken off the warp is the loading. The
// [outer*len, inner] input is described to the TMA engine as a 2-D tensor; lane 0 keeps COLS_STAGES
// tile copies of [128 rows x 32 columns] (16 KiB) in flight into a shared-memory ring, each completing
// on an mbarrier, and the warp walks a landed tile row by row, lane = column (conflict-free). No other
// warps, no CTA barriers. Tiles that reach past the tensor (or past `inner`) are zero-filled by the
// hardware and those rows / columns are simply not consumed. Waits are bounded as in the row kernel.
// Tile height: 128 rows (16 KiB tiles, 64 KiB ring, three CTAs per SM) when there are CTAs to spare;
// 256 rows (the TMA box limit; 128 KiB ring) when the column groups are fewer than two per SM, which
// halves the per-tile bookkeeping of the one warp that does everything.
constexpr int COLS_STAGES = 4;
constexpr size_t cols_smem(int tile_rows) { return (size_t)COLS_STAGES * tile_rows * 128 + 8 * 128; }  // + 8 rows of slack for look-ahead loads

__device__ __forceinline__ void tile_load_2d(void *dst, const CUtensorMap *map, int32_t x, int32_t y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_addr(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
                 : "memory");
}

template <int COLS_TILE_ROWS>
__global__ void __launch_bounds__(32) sum_cols_tma_kernel(const __grid_constant__ CUtensorMap map, uint64_t len, uint64_t inner,
                                                          uint32_t groups_per_outer, float *__restrict__ out, int *status) {
    ordered_start();
    constexpr uint32_t COLS_TILE_BYTES = COLS_TILE_ROWS * 32 * sizeof(float);
    extern __shared__ __align__(128) unsigned char cols_ring[];
    __shared__ uint64_t bars[COLS_STAGES];
    float *ring = reinterpret_cast<float *>(cols_ring);  // [COLS_STAGES][COLS_TILE_ROWS][32]
    const int lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < COLS_STAGES; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const uint64_t o = blockIdx.x / groups_per_outer;
    const uint32_t c0 = (blockIdx.x % groups_per_outer) * 32;
    const uint32_t ncols = inner - c0 < 32 ? (uint32_t)(inner - c0) : 32;
    const uint64_t row0 = o * len;  // first row of this slab in the 2-D view
    const uint32_t tiles = (uint32_t)((len + COLS_TILE_ROWS - 1) / COLS_TILE_ROWS);
    if (lane == 0) {
        for (uint32_t t = 0; t < COLS_STAGES && t < tiles; ++t) {
            mbar_expect_tx(&bars[t], COLS_TILE_BYTES);
            tile_load_2d(ring + (size_t)t * COLS_TILE_ROWS * 32, &map, (int32_t)c0, (int32_t)(row0 + (uint64_t)t * COLS_TILE_ROWS), &bars[t]);
        }
    }
    float s = 0.0f;
    for (uint32_t t = 0; t < tiles; ++t) {
        const int st = t % COLS_STAGES;
        if (!mbar_wait_bounded(&bars[st], (t / COLS_STAGES) & 1)) {
            for (uint32_t d = t + 1; d < tiles && d < t + COLS_STAGES; ++d) (void)mbar_wait_bounded(&bars[d % COLS_STAGES], (d / COLS_STAGES) & 1);
            if (lane == 0) {
                *(volatile int *)status = STATUS_WAIT_EXPIRED;
                __threadfence_system();
            }
            return;
        }
        const float *buf = ring + (size_t)st * COLS_TILE_ROWS * 32 + lane;
        const uint32_t rows = (uint32_t)(len - (uint64_t)t * COLS_TILE_ROWS < COLS_TILE_ROWS ? len - (uint64_t)t * COLS_TILE_ROWS : COLS_TILE_ROWS);
        // One warp, one dependent add per row: the loop must cost little more than the add latency.
        // The shared-memory load of row r+8 is issued between the adds of rows r and r+1 (volatile asm
        // pins that order), so loads ride in the adds' latency shadow instead of running in batches.
        uint32_t r = 0;
        if (rows >= 32) {
            const uint32_t addr = smem_addr(buf);
            float v[40];
#pragma unroll
            for (int u = 0; u < 8; ++u) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[u]) : "r"(addr + u * 128));
            for (; r + 32 <= rows; r += 32) {
                const uint32_t a = addr + r * 128;
#pragma unroll
                for (int u = 0; u < 32; ++u) {
                    // rows past the tile's end are never added; the address stays inside the ring
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[(u + 8) % 40]) : "r"(a + (u + 8) * 128));
                    s = __fadd_rn(s, v[u]);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = v[32 + u];
            }
        }
        for (; r < rows; ++r) s = __fadd_rn(s, buf[r * 32]);
        __syncwarp();  // every lane is done with this stage before it is refilled
        if (lane == 0 && t + COLS_STAGES < tiles) {
            mbar_expect_tx(&bars[st], COLS_TILE_BYTES);
            tile_load_2d(ring + (size_t)st * COLS_TILE_ROWS * 32, &map, (int32_t)c0, (int32_t)(row0 + (uint64_t)(t + COLS_STAGES) * COLS_TILE_ROWS), &bars[st]);
        }
    }
    if (lane < (int)ncols) out[o * inner + c0 + lane] = s;
}

// inner > 1, TMA-staged, chains fed by ldmatrix: the form that brings a column's chain down to the add
// latency. In the kernel above the warp that owns the chains fetches every row with one 4-byte
// shared-memory load, and a lone warp cannot issue a load and a dependent add in the same four
// cycles: 5.1 to 6.3 cycles per row measured on the bare loop, 7.5 in that kernel, against 4.07 for the
// dependent adds alone. What the chain of column c needs is rows r, r+1, r+2, r+3 of column c in four
// registers of lane c. That is exactly what ldmatrix.x4 delivers when it is pointed at four
// consecutive 128-byte rows of the row-major tile as the TMA engine lands it: a "matrix" of eight
// 16-byte rows is one 128-byte tile row (eight chunks of four columns), and the instruction hands
// thread T the 32-bit element (matrix row T / 4, position T % 4), i.e. column 4 (T / 4) + T % 4 = T of that
// tile row. One instruction per four rows, no transposition, no extra shared-memory traffic: 4.29
// cycles per row measured on the bare loop.
//   * warp 1, one lane (producer): keeps STAGES tile copies of [128 rows x 32 columns] in flight and
//     refills a stage when the chain warp has released it;
//   * warp 0 (chains): adds the rows of its column in row order from 0.0 as the reference does
//     (reduce.rs:132-145), sixteen rows of loads always in flight ahead of the adds, across tile
//     boundaries too.
// Every wait is bounded; a wait that runs out is reported through *status, the copies that may still
// be in flight get the same bounded chance to land, and the CTA exits without a result.
constexpr size_t ldm_smem(int stages, int rows) { return 128 /* alignment slack */ + (size_t)stages * rows * 128 + 2 * stages * sizeof(uint64_t) + 16; }

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Rows r .. r+3 of the lane's column, from four consecutive 128-byte rows of a row-major f32 tile:
// `addr` = tile row r + lane / 8, 16-byte chunk lane % 8 (the row address every thread supplies).
__device__ __forceinline__ float4 ldmatrix_rows4(uint32_t addr) {
    float4 v;
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

template <int STAGES, int LDM_ROWS>
__global__ void __launch_bounds__(64) sum_cols_ldm_kernel(const __grid_constant__ CUtensorMap map, uint64_t len, uint64_t inner,
                                                          uint32_t groups_per_outer, float *__restrict__ out, int *status) {
    ordered_start();
    constexpr uint32_t LDM_TILE_BYTES = LDM_ROWS * 32 * sizeof(float);
    extern __shared__ unsigned char ldm_raw[];
    const uint32_t base = (smem_addr(ldm_raw) + 127u) & ~127u;
    unsigned char *aligned = ldm_raw + (base - smem_addr(ldm_raw));
    float *ring = reinterpret_cast<float *>(aligned);  // [STAGES][128][32]
    uint64_t *full = reinterpret_cast<uint64_t *>(aligned + (size_t)STAGES * LDM_TILE_BYTES), *empty = full + STAGES;
    volatile int *failed = reinterpret_cast<volatile int *>(empty + STAGES);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * STAGES; ++i) mbar_init(&full[i], 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint64_t o = blockIdx.x / groups_per_outer;
    const uint32_t c0 = (blockIdx.x % groups_per_outer) * 32;
    const uint32_t ncols = inner - c0 < 32 ? (uint32_t)(inner - c0) : 32;
    const uint64_t row0 = o * len;
    const uint32_t tiles = (uint32_t)((len + LDM_ROWS - 1) / LDM_ROWS), full_tiles = (uint32_t)(len / LDM_ROWS);

    if (warp == 1) {
        // ---- producer: one lane ----
        if (lane != 0) return;
        for (uint32_t t = 0; t < tiles; ++t) {
            const int st = t % STAGES;
            if (t >= (uint32_t)STAGES && !mbar_wait_bounded(&empty[st], ((t / STAGES) - 1) & 1)) {
                *failed = 1;
                *(volatile int *)status = STATUS_WAIT_EXPIRED;
                __threadfence_system();
                return;
            }
            if (*failed) return;
            mbar_expect_tx(&full[st], LDM_TILE_BYTES);
            tile_load_2d(ring + (size_t)st * LDM_ROWS * 32, &map, (int32_t)c0, (int32_t)(row0 + (uint64_t)t * LDM_ROWS), &full[st]);
        }
        return;
    }

    // ---- chains ----
    const uint32_t lane_off = (uint32_t)(lane >> 3) * 128 + (uint32_t)(lane & 7) * 16;
    constexpr uint32_t NONE = 0xffffffffu;
    uint32_t gave_up_at = NONE;  // the tile whose wait ran out, if any
    float s = 0.0f;
    float4 v[2][4];  // two batches of sixteen rows: one being added, one in flight
    if (full_tiles > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full[0], 0))) gave_up_at = 0;
        const uint32_t a0 = smem_addr(ring) + lane_off;
#pragma unroll
        for (int u = 0; u < 4; ++u) v[0][u] = ldmatrix_rows4(a0 + 4 * u * 128);
    }
    for (uint32_t t = 0; t < full_tiles && gave_up_at == NONE; ++t) {
        const uint32_t a = smem_addr(ring + (size_t)(t % STAGES) * LDM_ROWS * 32) + lane_off;
        const uint32_t nt = t + 1;
        bool next_landed = false;
#pragma unroll
        for (int bb = 0; bb < LDM_ROWS / 16; ++bb) {
            // One look at the next tile's barrier well before it is needed: the answer is back by the time
            // the last batch of this tile is reached, and the wait below is then skipped.
            if (bb == LDM_ROWS / 16 - 3 && nt < full_tiles) next_landed = mbar_try_wait(&full[nt % STAGES], (nt / STAGES) & 1);
            if (bb + 1 < LDM_ROWS / 16) {
#pragma unroll
                for (int u = 0; u < 4; ++u) v[(bb + 1) & 1][u] = ldmatrix_rows4(a + (16 * (bb + 1) + 4 * u) * 128);
            } else if (nt < full_tiles) {  // the next tile's first sixteen rows (it has normally landed long ago)
                if (!__all_sync(0xffffffffu, next_landed) && !__all_sync(0xffffffffu, mbar_wait_bounded(&full[nt % STAGES], (nt / STAGES) & 1)))
                    gave_up_at = nt;
                const uint32_t an = smem_addr(ring + (size_t)(nt % STAGES) * LDM_ROWS * 32) + lane_off;
#pragma unroll
                for (int u = 0; u < 4; ++u) v[0][u] = ldmatrix_rows4(an + 4 * u * 128);  // harmless if the wait ran out: the result is dropped
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                s = __fadd_rn(s, v[bb & 1][u].x);
                s = __fadd_rn(s, v[bb & 1][u].y);
                s = __fadd_rn(s, v[bb & 1][u].z);
                s = __fadd_rn(s, v[bb & 1][u].w);
            }
        }
        __syncwarp();  // every lane has its last rows of this stage in registers
        if (lane == 0) mbar_arrive(&empty[t % STAGES]);
    }
    if (full_tiles < tiles && gave_up_at == NONE) {  // the last, partial tile: row by row (rows past the end were zero-filled and are not added)
        const uint32_t t = full_tiles;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full[t % STAGES], (t / STAGES) & 1))) {
            gave_up_at = t;
        } else {
            const float *buf = ring + (size_t)(t % STAGES) * LDM_ROWS * 32 + lane;
            const uint32_t rows = (uint32_t)(len - (uint64_t)t * LDM_ROWS);
            for (uint32_t r = 0; r < rows; ++r) s = __fadd_rn(s, buf[r * 32]);
        }
    }
    if (gave_up_at != NONE) {
        // A wait that ran out: tell the producer, give the copies it may have issued (at most STAGES - 1
        // tiles past that one) their bounded chance to land, report, leave without a result.
        if (lane == 0) *failed = 1;
        for (uint32_t d = gave_up_at + 1; d < tiles && d < gave_up_at + STAGES; ++d) (void)mbar_wait_bounded(&full[d % STAGES], (d / STAGES) & 1);
        if (lane == 0) {
            *(volatile int *)status = STATUS_WAIT_EXPIRED;
            __threadfence_system();
        }
        return;
    }
    if (lane < (int)ncols) out[o * inner + c0 + lane] = s;
}

// ---- max / argmax ---------------------------------------------------------------------------------------

// Should candidate (v, i) replace the current best (bv, bi)? NaN beats every number; among equals
// (or among NaNs) the lower index wins.
__device__ __forceinline__ bool vi_better(float v, uint64_t i, float bv, uint64_t bi) {
    const bool vn = v != v, bn = bv != bv;
    if (vn || bn) return vn && (!bn || i < bi);
    return v > bv || (v == bv && i < bi);
}

// Scanning in increasing index order: strictly greater replaces; a NaN replaces a non-NaN.
__device__ __forceinline__ void scan_step(float v, uint64_t i, float &bv, uint64_t &bi) {
    if (v > bv || (v != v && bv == bv)) {
        bv = v;
        bi = i;
    }
}

constexpr int MAX_CTA = 256;
constexpr int MAX_UNROLL = 4;

// The max/argmax counterpart of the sum's in-launch combine: CTA 0 gathers the segment maxima that the
// worker CTAs publish through the mailbox ((epoch << 32) | float bits, stored with release semantics
// AFTER the segment's position has been written to `seg_pos`), keeps the best (value, segment) pair -
// NaN wins, then the larger value, then the lower segment - and writes the row's result. Max is
// order-free, so all 256 threads poll and scan in parallel; polls are bounded.
__device__ void max_combiner_body(const unsigned long long *mailbox, uint32_t epoch, uint64_t segs, const int64_t *seg_pos, float *out_v,
                                  int64_t *out_i, int64_t idx_offset, int *status, const PeerXchg &px) {
    __shared__ float sv[8];
    __shared__ uint64_t ss[8];
    constexpr int WORDS = 8;
    float bv = __int_as_float(0xff800000);
    uint64_t bs = ~0ull;
    bool failed = false;
    for (uint64_t base = 0; base < segs; base += (uint64_t)MAX_CTA * WORDS) {
        float v[WORDS];
        uint32_t missing = 0;
#pragma unroll
        for (int k = 0; k < WORDS; ++k)
            if (base + (uint64_t)k * MAX_CTA + threadIdx.x < segs) missing |= 1u << k;
        const uint32_t mine = missing;
        for (uint32_t tries = 0; tries < POLL_LIMIT && missing; ++tries) {
#pragma unroll
            for (int k = 0; k < WORDS; ++k)
                if (missing & (1u << k)) {
                    unsigned long long w;
                    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(mailbox + base + (uint64_t)k * MAX_CTA + threadIdx.x) : "memory");
                    if ((uint32_t)(w >> 32) == epoch) {
                        v[k] = __uint_as_float((uint32_t)w);
                        missing &= ~(1u << k);
                    }
                }
        }
        failed = failed || missing != 0;
#pragma unroll
        for (int k = 0; k < WORDS; ++k)
            if ((mine & ~missing) & (1u << k)) {
                const uint64_t seg = base + (uint64_t)k * MAX_CTA + threadIdx.x;
                if (bs == ~0ull) bs = seg;  // first segment this thread sees: position even if its value is -inf
                scan_step(v[k], seg, bv, bs);
            }
    }
    if (__syncthreads_or(failed)) {
        if (threadIdx.x == 0) {
            *(volatile int *)status = STATUS_WAIT_EXPIRED;
            __threadfence_system();
        }
        return;
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
        const uint64_t os = __shfl_xor_sync(0xffffffffu, bs, d);
        if (vi_better(ov, os, bv, bs)) { bv = ov; bs = os; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; ss[threadIdx.x >> 5] = bs; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = threadIdx.x < 8 ? sv[threadIdx.x] : __int_as_float(0xff800000);
        bs = threadIdx.x < 8 ? ss[threadIdx.x] : ~0ull;
#pragma unroll
        for (int d = 4; d >= 1; d >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
            const uint64_t os = __shfl_xor_sync(0xffffffffu, bs, d);
            if (vi_better(ov, os, bv, bs)) { bv = ov; bs = os; }
        }
        if (px.world > 0) {  // lanes 0-7 hold the row's best pair; hand lane 0's to the whole warp
            bv = __shfl_sync(0xffffffffu, bv, 0);
            bs = __shfl_sync(0xffffffffu, bs, 0);
            // Without positions, the rank stands in for one: equal maxima (+0 and -0, two NaNs) then resolve
            // to the lower rank, as a scan over the per-rank results in rank order would.
            const int64_t pos = out_i ? seg_pos[bs] + idx_offset : (int64_t)px.rank;
            return peer_finish(px, out_i ? REDUCE_MAX_ARGMAX : REDUCE_MAX, bv, pos, out_v, out_i, status);
        }
        if (threadIdx.x == 0) {
            if (out_i) out_i[0] = seg_pos[bs] + idx_offset;
            if (out_v) out_v[0] = bv;
        }
    }
}

__device__ void max_combiner(const unsigned long long *mailbox, uint32_t epoch, uint64_t segs, const int64_t *seg_pos, float *out_v, int64_t *out_i,
                             int64_t idx_offset, int *status, const PeerXchg &px, unsigned long long *done, uint32_t lag) {
    combiner_begin(done, epoch, status, lag);  // same ordering rules as the sum's combiner
    max_combiner_body(mailbox, epoch, segs, seg_pos, out_v, out_i, idx_offset, status, px);
    __syncthreads();
    if (threadIdx.x == 0) combiner_end(done, epoch);
}

// What a fused launch adds to max_rows_kernel's arguments (mailbox == nullptr: the plain two-pass form).
struct MaxFused {
    unsigned long long *mailbox;
    uint32_t epoch;
    float *final_v;
    int64_t *final_i;
    int64_t final_offset;
    int *status;
    PeerXchg px;
    int ordered;  // workers wait for the kernel before this one to complete before they read (see sum_rows_tma_kernel)
    unsigned long long *done;  // the device's word of finished launch numbers (see combiner_begin)
};

// inner == 1. Task t = (row, seg): elements [seg*seg_len, min(len, (seg+1)*seg_len)) of row. TPT
// threads share one task (32: a warp per task, 256: the CTA). VEC 4 requires every task start to be
// 16-byte aligned (the host guarantees it). Writes the value and/or (ARG) the index within the row
// plus idx_offset, whichever output pointers are not null.
template <int TPT, int VEC, bool ARG>
__global__ void __launch_bounds__(MAX_CTA) max_rows_kernel(const float *__restrict__ x, uint64_t tasks, uint64_t len,
                                                           uint64_t segs, uint64_t seg_len, float *__restrict__ out_v,
                                                           int64_t *__restrict__ out_i, int64_t idx_offset, const __grid_constant__ MaxFused fused) {
    constexpr int PER_CTA = MAX_CTA / TPT;
    if (TPT == MAX_CTA && fused.mailbox != nullptr && blockIdx.x == 0)
        return max_combiner(fused.mailbox, fused.epoch, segs, out_i, fused.final_v, fused.final_i, fused.final_offset, fused.status, fused.px, fused.done, (uint32_t)fused.ordered >> 8);
    if (TPT == MAX_CTA && fused.mailbox != nullptr && !(fused.ordered & 1)) launch_dependents();
    else ordered_start();
    const uint64_t cta = (TPT == MAX_CTA && fused.mailbox != nullptr) ? blockIdx.x - 1 : blockIdx.x;
    const uint64_t t = cta * PER_CTA + threadIdx.x / TPT;
    const int lane = threadIdx.x % TPT;
    const bool live = t < tasks;
    // Every thread starts from (-inf, first index it will look at), so a slice of nothing but -inf
    // still reports its first position; a thread with nothing to look at holds (-inf, ~0).
    float bv = __int_as_float(0xff800000);
    uint64_t bi = ~0ull;
    if (live) {
        const uint64_t row = t / segs, seg = t - row * segs;
        const uint64_t lo = seg * seg_len;
        const uint64_t hi = lo + seg_len < len ? lo + seg_len : len;
        const float *p = x + row * len;
        if constexpr (VEC == 4) {
            const uint64_t vend = lo + ((hi - lo) & ~3ull);
            uint64_t i = lo + (uint64_t)lane * 4;
            if (i < vend) bi = i;
            else if (lane == 0 && vend < hi) bi = vend;
            for (; i + (uint64_t)(MAX_UNROLL - 1) * TPT * 4 < vend; i += (uint64_t)MAX_UNROLL * TPT * 4) {
                float4 v[MAX_UNROLL];
#pragma unroll
                for (int u = 0; u < MAX_UNROLL; ++u) v[u] = ldf4(p + i + (uint64_t)u * TPT * 4);
#pragma unroll
                for (int u = 0; u < MAX_UNROLL; ++u) {
                    const uint64_t j = i + (uint64_t)u * TPT * 4;
                    scan_step(v[u].x, j, bv, bi);
                    scan_step(v[u].y, j + 1, bv, bi);
                    scan_step(v[u].z, j + 2, bv, bi);
                    scan_step(v[u].w, j + 3, bv, bi);
                }
            }
            for (; i < vend; i += (uint64_t)TPT * 4) {
                const float4 v = ldf4(p + i);
                scan_step(v.x, i, bv, bi);
                scan_step(v.y, i + 1, bv, bi);
                scan_step(v.z, i + 2, bv, bi);
                scan_step(v.w, i + 3, bv, bi);
            }
            if (lane == 0)
                for (uint64_t j = vend; j < hi; ++j)
                    if (vi_better(p[j], j, bv, bi)) { bv = p[j]; bi = j; }
        } else {
            if (lo + lane < hi) bi = lo + lane;
            for (uint64_t i = lo + lane; i < hi; i += TPT) scan_step(ldf(p + i), i, bv, bi);
        }
    }
    // (-inf, ~0) loses every comparison against a real element: equal values resolve to the lower index.
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
        const uint64_t oi = __shfl_xor_sync(0xffffffffu, bi, d);
        if (vi_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if constexpr (TPT > 32) {
        __shared__ float sv[TPT / 32];
        __shared__ uint64_t si[TPT / 32];
        if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
        __syncthreads();
        if (threadIdx.x < 32) {
            bv = threadIdx.x < TPT / 32 ? sv[threadIdx.x] : __int_as_float(0xff800000);
            bi = threadIdx.x < TPT / 32 ? si[threadIdx.x] : ~0ull;
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
                const uint64_t oi = __shfl_xor_sync(0xffffffffu, bi, d);
                if (vi_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
        }
    }
    if (live && lane == 0) {
        if (TPT == MAX_CTA && fused.mailbox != nullptr) {
            if (ARG && out_i) out_i[t] = (int64_t)bi;  // position within the row, read by the combiner after the acquire
            const unsigned long long w = ((unsigned long long)fused.epoch << 32) | __float_as_uint(bv);
            asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(fused.mailbox + t), "l"(w) : "memory");
        } else {
            if (out_v) out_v[t] = bv;
            if (ARG && out_i) out_i[t] = (int64_t)bi + idx_offset;
        }
    }
}

// Pass 2 for rows split into several segments: a CTA per row. Each thread scans a strided share of
// the row's segment results, then the CTA picks the best (value, segment) pair: the lowest segment
// wins ties, so the lowest position does. Writes the value and/or the index (plus idx_offset),
// whichever output pointers are not null.
__global__ void __launch_bounds__(256) max_combine_kernel(const float *__restrict__ pv, const int64_t *__restrict__ pi, uint64_t outer,
                                                          uint64_t segs, float *__restrict__ out_v, int64_t *__restrict__ out_i,
                                                          int64_t idx_offset) {
    ordered_start();
    __shared__ float sv[8];
    __shared__ uint64_t ss[8];
    const uint64_t r = blockIdx.x;
    float bv = __int_as_float(0xff800000);
    uint64_t bs = threadIdx.x < segs ? threadIdx.x : ~0ull;
    for (uint64_t s = threadIdx.x; s < segs; s += 256) scan_step(pv[r * segs + s], s, bv, bs);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
        const uint64_t os = __shfl_xor_sync(0xffffffffu, bs, d);
        if (vi_better(ov, os, bv, bs)) { bv = ov; bs = os; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; ss[threadIdx.x >> 5] = bs; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = threadIdx.x < 8 ? sv[threadIdx.x] : __int_as_float(0xff800000);
        bs = threadIdx.x < 8 ? ss[threadIdx.x] : ~0ull;
#pragma unroll
        for (int d = 4; d >= 1; d >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
            const uint64_t os = __shfl_xor_sync(0xffffffffu, bs, d);
            if (vi_better(ov, os, bv, bs)) { bv = ov; bs = os; }
        }
        if (threadIdx.x == 0) {
            if (out_i) out_i[r] = pi[r * segs + bs] + idx_offset;
            if (out_v) out_v[r] = bv;
        }
    }
}

// inner > 1: thread per output column scans rows j in order.
__global__ void __launch_bounds__(256) max_cols_kernel(const float *__restrict__ x, uint64_t total, uint64_t len, uint64_t inner,
                                                       float *__restrict__ out_v, int64_t *__restrict__ out_i, int64_t idx_offset) {
    ordered_start();
    const uint64_t t = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (t >= total) return;
    const uint64_t o = t / inner, i = t - o * inner;
    const float *p = x + o * len * inner + i;
    float bv = ldf(p);
    uint64_t bi = 0;
    uint64_t j = 1;
    for (; j + COL_UNROLL <= len; j += COL_UNROLL) {
        float v[COL_UNROLL];
#pragma unroll
        for (int u = 0; u < COL_UNROLL; ++u) v[u] = ldf(p + (j + u) * inner);
#pragma unroll
        for (int u = 0; u < COL_UNROLL; ++u) scan_step(v[u], j + u, bv, bi);
    }
    for (; j < len; ++j) scan_step(ldf(p + j * inner), j, bv, bi);
    if (out_i) out_i[t] = (int64_t)bi + idx_offset;
    if (out_v) out_v[t] = bv;
}

// Combine of a sharded argmax: vals/idx are [g, m], one row of candidates per shard; per column the
// best candidate's position is kept (NaN wins, then the larger value, then the lower position).
__global__ void __launch_bounds__(256) argmax_combine_kernel(const float *__restrict__ vals, const int64_t *__restrict__ idx, uint64_t g,
                                                             uint64_t m, int64_t *__restrict__ out) {
    ordered_start();
    const uint64_t j = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (j >= m) return;
    float bv = vals[j];
    uint64_t bi = (uint64_t)idx[j];
    for (uint64_t r = 1; r < g; ++r) {
        const float v = vals[r * m + j];
        const uint64_t i = (uint64_t)idx[r * m + j];
        if (vi_better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    out[j] = (int64_t)bi;
}

// ---- host-side planning ------------------------------------------------------------------------------------

struct MaxPlan {
    int tpt;           // threads per task: 32 or 256
    int vec;           // 1 or 4
    uint64_t segs;     // segments per row
    uint64_t seg_len;  // elements per segment (multiple of 4)
};

MaxPlan plan_max(uint64_t outer, uint64_t len, int /*sms*/) {
    MaxPlan m;
    m.vec = (len % 4 == 0 || outer == 1) ? 4 : 1;
    if (len <= 16384) {
        m.tpt = 32;
        m.segs = 1;
        m.seg_len = (len + 3) & ~3ull;
        return m;
    }
    // Long rows: a 256-thread CTA per 16384-element segment (four batches of four float4 per thread).
    // Measured on a 1 GiB row: segments of 8 Ki to 256 Ki elements all run within 3% of each other and
    // 16 Ki is the best; 4 Ki pays too much per-CTA epilogue, 1 Mi leaves too few CTAs.
    m.tpt = 256;
    m.seg_len = 16384;
    m.segs = (len + m.seg_len - 1) / m.seg_len;
    return m;
}

}  // namespace

// One word per device of pinned, device-visible host memory in which that device's kernels report a
// bounded wait that ran out (0 = nothing to report). Written by the device, taken (read and cleared in
// one atomic exchange) by the host at the next blocking call on that device, so a report is delivered
// exactly once and to the device it belongs to, whichever threads drive the devices.
int *reduce_status_word(int device) {
    static int *words = [] {
        int *p = nullptr;
        if (cudaHostAlloc((void **)&p, 64 * sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
            (void)cudaGetLastError();
            return (int *)nullptr;
        }
        for (int i = 0; i < 64; ++i) p[i] = 0;
        return p;
    }();
    return words && device >= 0 && device < 64 ? words + device : nullptr;
}

int take_reduce_status(int device) {
    int *w = reduce_status_word(device);
    return w ? __atomic_exchange_n(w, 0, __ATOMIC_ACQ_REL) : 0;
}

namespace {
// The in-launch combiners' mailbox: MAILBOX_REGIONS regions per device, each MAILBOX_SLOTS 64-bit
// value words followed by as many 64-bit position words (the max/argmax combiner reads a segment's
// position there), allocated and zeroed on first use and kept for the life of the process. Each
// launch gets the next epoch (never 0) and the region epoch mod MAILBOX_REGIONS: launch e+4 starts
// only after the combiner of e+1 has finished, which is after launch e has completed (see
// combiner_begin), so a region is not written again before its last reader is done. The word after
// the regions is `done`, the number of the newest launch whose combiner has finished. When the 32-bit epoch wraps the words are zeroed again, on the stream, so no stale
// word can match.
constexpr uint64_t MAILBOX_SLOTS = 1ull << 18;  // a sum's row of up to 2^34 elements, a max's of up to 2^32
constexpr int MAILBOX_REGIONS = 4;
constexpr size_t MAILBOX_BYTES = (size_t)MAILBOX_REGIONS * MAILBOX_SLOTS * 2 * 8 + 256;  // + the word of finished launch numbers
// PYTORCHES_B200_FUSED_COMBINE=0 in the environment turns the in-launch combines off (two launches
// per reduction instead of one); a diagnostic switch, read once.
unsigned long long *mailbox_for(int device, cudaStream_t s, uint32_t *epoch, unsigned long long **done) {
    static const bool enabled = [] {
        const char *e = getenv("PYTORCHES_B200_FUSED_COMBINE");
        return !(e && e[0] == '0');
    }();
    if (!enabled) return nullptr;
    static std::mutex mu;
    static unsigned long long *box[64] = {};
    static uint32_t next[64] = {};
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!box[device]) {
        void *p = nullptr;
        if (cudaMalloc(&p, MAILBOX_BYTES) != cudaSuccess || cudaMemsetAsync(p, 0, MAILBOX_BYTES, s) != cudaSuccess) {
            (void)cudaGetLastError();
            if (p) (void)cudaFree(p);
            return nullptr;
        }
        box[device] = (unsigned long long *)p;
    }
    if (++next[device] == 0) {
        if (cudaMemsetAsync(box[device], 0, MAILBOX_BYTES, s) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        next[device] = 1;
    }
    *epoch = next[device];
    *done = box[device] + (size_t)MAILBOX_REGIONS * MAILBOX_SLOTS * 2;
    return box[device] + (size_t)(next[device] % MAILBOX_REGIONS) * MAILBOX_SLOTS * 2;
}

}  // namespace

// PYTORCHES_B200_OVERLAP=0 turns early scheduling and the early start of back-to-back reductions off
// (every kernel is then launched the ordinary way; diagnostic, read once).
bool overlap_enabled() {
    static const bool enabled = [] {
        const char *e = getenv("PYTORCHES_B200_OVERLAP");
        return !(e && e[0] == '0');
    }();
    return enabled;
}

namespace {
// The staged row sum's ring shapes (stages, floats per copy). pick_ring chooses by the number of
// worker CTAs: see the comment at TMA_MIN_CHUNK. PYTORCHES_B200_SUM_RING=<index> forces one (diagnostic).
struct RingShape { int stages; uint32_t chunk; };
constexpr RingShape RINGS[] = {{4, 4096}, {2, 4096}, {3, 4096}, {4, 2048}, {2, 8192}};
constexpr int N_RINGS = sizeof(RINGS) / sizeof(RINGS[0]);
int pick_ring(uint64_t tasks, int sms) {
    static const int forced = [] {
        const char *e = getenv("PYTORCHES_B200_SUM_RING");
        return e && e[0] >= '0' && e[0] < '0' + N_RINGS ? e[0] - '0' : -1;
    }();
    if (forced >= 0) return forced;
    return tasks <= (uint64_t)sms * 12 ? 1 : 0;
}

// Opts the staged kernels into their 64 KiB of dynamic shared memory, once per device.
bool staged_kernels_ready(int device) {
    static std::mutex mu;
    static bool done[64] = {}, ok[64] = {};
    if (device < 0 || device >= 64) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[device]) {
        done[device] = true;
        bool good = true;
#define B200_RING_ATTR(I)                                                                                                              \
    good = good &&                                                                                                                     \
           cudaFuncSetAttribute(sum_rows_tma_kernel<false, RINGS[I].stages, RINGS[I].chunk>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                (int)ring_bytes(RINGS[I].stages, RINGS[I].chunk)) == cudaSuccess &&                                    \
           cudaFuncSetAttribute(sum_rows_tma_kernel<true, RINGS[I].stages, RINGS[I].chunk>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                (int)fused_smem(RINGS[I].stages, RINGS[I].chunk, true)) == cudaSuccess;
        B200_RING_ATTR(0) B200_RING_ATTR(1) B200_RING_ATTR(2) B200_RING_ATTR(3) B200_RING_ATTR(4)
#undef B200_RING_ATTR
        ok[device] = good &&
                     cudaFuncSetAttribute(sum_cols_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cols_smem(128)) == cudaSuccess &&
                     cudaFuncSetAttribute(sum_cols_tma_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cols_smem(256)) == cudaSuccess &&
                     cudaFuncSetAttribute(sum_cols_ldm_kernel<4, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ldm_smem(4, 256)) == cudaSuccess &&
                     cudaFuncSetAttribute(sum_cols_ldm_kernel<4, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ldm_smem(4, 128)) == cudaSuccess;
        if (!ok[device]) (void)cudaGetLastError();
    }
    return ok[device];
}

// Describes x, viewed as a row-major [rows, inner] f32 matrix, to the TMA engine with tiles of
// [COLS_TILE_ROWS x 32]. The encoder lives in the driver; it is looked up through the runtime so that
// this library still has no link-time dependency on libcuda. False if it is unavailable or refuses.
// Tiles are [tile_rows x 32].
bool make_cols_tensor_map(CUtensorMap *map, const float *x, uint64_t rows, uint64_t inner, uint32_t tile_rows) {
    using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            fn = nullptr;
        }
        return (EncodeFn)fn;
    }();
    if (!encode) return false;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {inner * sizeof(float)};
    const cuuint32_t box[2] = {32, tile_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)x, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

// ---- peer windows ------------------------------------------------------------------------------------------
// One window per device of this process: a 2 MiB allocation of its own (so that its IPC handle shares
// a driver allocation with nothing else): the scalar slots, then the vector area (see peer_vector_sum_kernel). It is
// created and zeroed by the first export and kept for the life of the process; every export zeroes it
// again, so that epochs may restart with a new group of ranks. Peers' windows are opened once per
// handle and never closed.
namespace {
constexpr size_t PEER_WINDOW_BYTES = size_t(4) << 20;
static_assert(PEER_WINDOW_WORDS <= PEER_VECTOR_AREA_WORD, "the scalar slots end before the vector area");
static_assert((PEER_BLOCK_AREA_WORD + (size_t)PEER_GENERATIONS * PEER_BLOCKS_MAX) * 8 <= PEER_WINDOW_BYTES, "the vector and block areas fit the window");
struct PeerWindows {
    std::mutex mu;
    unsigned long long *local[64] = {};
    unsigned long long *trace[64] = {};  // PEER_TRACE_RECORDS x PEER_TRACE_WORDS words per device
    cudaIpcMemHandle_t local_handle[64] = {};
    std::vector<std::pair<cudaIpcMemHandle_t, void *>> opened[64];
    PeerXchg attached[64] = {};
};
PeerWindows &peer_windows() {
    static PeerWindows w;
    return w;
}
}  // namespace

cudaError_t peer_window_export(int device, void *handle, cudaStream_t s) {
    if (device < 0 || device >= 64 || !handle) return cudaErrorInvalidValue;
    PeerWindows &w = peer_windows();
    std::lock_guard<std::mutex> lock(w.mu);
    cudaError_t e;
    if (!w.local[device]) {
        void *p = nullptr;
        if ((e = cudaMalloc(&p, PEER_WINDOW_BYTES)) != cudaSuccess) return e;
        if ((e = cudaIpcGetMemHandle(&w.local_handle[device], p)) != cudaSuccess) {
            (void)cudaFree(p);
            return e;
        }
        w.local[device] = (unsigned long long *)p;
    }
    if (!w.trace[device]) {
        void *t = nullptr;
        if ((e = cudaMalloc(&t, (size_t)PEER_TRACE_RECORDS * PEER_TRACE_WORDS * 8)) != cudaSuccess) return e;
        w.trace[device] = (unsigned long long *)t;
    }
    if ((e = cudaMemsetAsync(w.trace[device], 0, (size_t)PEER_TRACE_RECORDS * PEER_TRACE_WORDS * 8, s)) != cudaSuccess) return e;
    w.attached[device] = PeerXchg{};
    // Everything this device has in flight finishes before the window is cleared, and the clearing
    // finishes before the handle leaves this call: no peer can write before it holds the handle.
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(w.local[device], 0, PEER_WINDOW_BYTES, s)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
    std::memcpy(handle, &w.local_handle[device], sizeof(cudaIpcMemHandle_t));
    return cudaSuccess;
}

cudaError_t peer_window_attach(int device, uint32_t rank, uint32_t world, const void *handles, uint32_t wait_ms) {
    if (device < 0 || device >= 64 || !handles || world == 0 || world > (uint32_t)PEER_MAX_RANKS || rank >= world) return cudaErrorInvalidValue;
    PeerWindows &w = peer_windows();
    std::lock_guard<std::mutex> lock(w.mu);
    if (!w.local[device]) return cudaErrorInvalidValue;  // export first
    PeerXchg px{};
    px.world = (int)world;
    px.rank = (int)rank;
    px.wait_ms = wait_ms ? wait_ms : 2000;
    // The trace is a diagnostic, off unless PYTORCHES_B200_PEER_TRACE=1: with several GPUs and sums in
    // unsplit order its few stores per reduction were measured to cost 10-40% of the step.
    static const bool tracing = [] {
        const char *e = getenv("PYTORCHES_B200_PEER_TRACE");
        return e && e[0] == '1';
    }();
    px.trace = tracing ? w.trace[device] : nullptr;
    for (uint32_t r = 0; r < world; ++r) {
        cudaIpcMemHandle_t h;
        std::memcpy(&h, (const char *)handles + (size_t)r * sizeof h, sizeof h);
        if (std::memcmp(&h, &w.local_handle[device], sizeof h) == 0) {  // this device's own window (rank r == rank, normally)
            px.window[r] = w.local[device];
            continue;
        }
        void *p = nullptr;
        for (auto &kv : w.opened[device])
            if (std::memcmp(&kv.first, &h, sizeof h) == 0) p = kv.second;
        if (!p) {
            cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) return e;
            w.opened[device].emplace_back(h, p);
        }
        px.window[r] = (unsigned long long *)p;
    }
    if (px.window[rank] != w.local[device]) return cudaErrorInvalidValue;  // handles[rank] must be this device's own
    w.attached[device] = px;
    return cudaSuccess;
}

// Copies the trace records of `device` (PEER_TRACE_RECORDS x PEER_TRACE_WORDS words) to the host.
cudaError_t peer_trace_read(int device, unsigned long long *out, cudaStream_t s) {
    if (device < 0 || device >= 64 || !out) return cudaErrorInvalidValue;
    PeerWindows &w = peer_windows();
    std::lock_guard<std::mutex> lock(w.mu);
    if (!w.trace[device]) return cudaErrorInvalidValue;
    cudaError_t e = cudaMemcpyAsync(out, w.trace[device], (size_t)PEER_TRACE_RECORDS * PEER_TRACE_WORDS * 8, cudaMemcpyDeviceToHost, s);
    return e == cudaSuccess ? cudaStreamSynchronize(s) : e;
}

bool peer_window_for(int device, uint64_t seq, PeerXchg *px) {
    if (device < 0 || device >= 64) return false;
    PeerWindows &w = peer_windows();
    std::lock_guard<std::mutex> lock(w.mu);
    if (w.attached[device].world <= 0) return false;
    *px = w.attached[device];
    px->epoch = (uint32_t)(seq % 0xfffffffeull) + 1;
    return true;
}

size_t reduce_scratch_bytes(ReduceKind kind, uint64_t outer, uint64_t len, uint64_t inner, int device) {
    if (inner != 1 || outer == 0 || len == 0) return 0;
    if (kind == REDUCE_SUM) {
        const uint64_t blocks = (len + SUM_BLOCK - 1) / SUM_BLOCK;
        return blocks > 1 ? outer * blocks * sizeof(float) : 0;
    }
    const MaxPlan m = plan_max(outer, len, sm_count(device));
    if (m.segs == 1) return 0;
    const uint64_t tasks = outer * m.segs;
    // values, then (16-byte aligned) indices
    return ((tasks * 4 + 15) & ~15ull) + (kind != REDUCE_MAX ? tasks * 8 : 0);
}

namespace {
bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

// May a reduction of [x, x + n) into out_v / out_i start while the reductions `c` describes are still
// finishing? Only if it touches nothing that they write and writes nothing that they touch.
bool may_overlap(const LaunchChain *c, const float *x, uint64_t n, const void *out_v, const void *out_i) {
    if (!c || !c->tail_open || !overlap_enabled()) return false;
    const char *lo = (const char *)x, *hi = lo + n * sizeof(float);
    for (const LaunchChain::Open *open : {&c->last, &c->before_last}) {
        for (const void *o : open->out) {
            if (!o) continue;
            if ((const char *)o >= lo && (const char *)o < hi) return false;  // it writes into our input
            if (o == out_v || o == out_i) return false;                       // both write the same word: order would matter
        }
        for (const void *o : {out_v, out_i})
            if (o && (const char *)o >= open->in_lo && (const char *)o < open->in_hi) return false;  // we write into its input
    }
    return true;
}

// How many launches back the combiner whose end a combiner awaits before it lets its successor start
// (see combiner_begin): 2, or 1 with PYTORCHES_B200_CHAIN_LAG=1 in the environment (a diagnostic).
uint32_t chain_lag() {
    static const uint32_t lag = [] {
        const char *e = getenv("PYTORCHES_B200_CHAIN_LAG");
        return e && e[0] == '1' ? 1u : 2u;
    }();
    return lag;
}

// `early`: this launch was allowed to start before `prev`'s newest one completed, so that one stays on the list.
void chain_opened(const LaunchChain *prev, LaunchChain *c, bool early, const float *x, uint64_t n, const void *out_v, const void *out_i) {
    if (!c) return;
    c->tail_open = true;
    c->before_last = early && prev ? prev->last : LaunchChain::Open{};
    c->last.in_lo = (const char *)x;
    c->last.in_hi = c->last.in_lo + n * sizeof(float);
    c->last.out[0] = out_v;
    c->last.out[1] = out_i;
}

// The local reduction. With `px`, a launch that ends in a combiner CTA also does the cross-GPU step
// there and sets *peer_done; every other path leaves it to the caller.
cudaError_t launch_reduce_local(ReduceKind kind, const float *x, uint64_t outer, uint64_t len, uint64_t inner, float *out_v, int64_t *out_i,
                                int64_t idx_offset, void *scratch, int device, cudaStream_t s, const PeerXchg *px, bool *peer_done,
                                const LaunchChain *prev, LaunchChain *next, float *spare_v) {
    const PeerXchg no_peers{};
    const uint64_t total = outer * inner;
    if (total == 0) return cudaSuccess;
    // Bulk copies and 128-bit loads need a 16-byte aligned base. Buffers of the plugin's allocator always
    // are; a pointer a host passes to an extension entry point need not be, and then the register-load
    // forms of the same kernels run (same order of operations, same bits).
    const bool base16 = aligned16(x);
    if (kind == REDUCE_SUM) {
        float *o = out_v;
        if (len == 0) return launch_fill(o, total, 0.0f, s);  // reduce.rs:106-109
        if (inner == 1) {
            if (len < 32) {
                B200_LAUNCH_ORDERED(sum_short_rows_kernel, (unsigned)((outer + 255) / 256), 256, 0, s, x, outer, (uint32_t)len, o);
                return cudaGetLastError();
            }
            const uint64_t blocks = (len + SUM_BLOCK - 1) / SUM_BLOCK, tasks = outer * blocks;
            float *dst = blocks == 1 ? o : (float *)scratch;
            // Long rows whose block starts are 16-byte aligned take the TMA-staged kernel.
            // A sum in unsplit order must take the one-launch form whatever its size: the other ranks wait for its block sums.
            const bool unsplit = px && px->blocks_total != 0;
            int *status = (base16 && (unsplit || len >= 8 * TMA_MIN_CHUNK) && (len % 4 == 0 || outer == 1) && tasks <= 0x7fffffffull) ? reduce_status_word(device) : nullptr;
            if (unsplit && !(status && outer == 1 && blocks <= MAILBOX_SLOTS && staged_kernels_ready(device))) return cudaErrorInvalidValue;
            if (status && staged_kernels_ready(device)) {
                // A single long row: chain the block sums inside the same launch (see ordered_combiner).
                uint32_t epoch = 0;
                unsigned long long *done = nullptr;
                unsigned long long *mailbox = (outer == 1 && (blocks >= 64 || unsplit) && blocks <= MAILBOX_SLOTS) ? mailbox_for(device, s, &epoch, &done) : nullptr;
                if (unsplit && !mailbox) return cudaErrorInvalidValue;
                const int ring = pick_ring(tasks, sm_count(device));
                const bool early = mailbox && may_overlap(prev, x, len, o, nullptr);
#define B200_RING_CASE(I)                                                                                                                   \
    if (ring == I) {                                                                                                                        \
        if (mailbox)                                                                                                                        \
            B200_LAUNCH_ORDERED((sum_rows_tma_kernel<true, RINGS[I].stages, RINGS[I].chunk>), (unsigned)tasks + (unsplit ? 2 : 1), 32,       \
                                fused_smem(RINGS[I].stages, RINGS[I].chunk, unsplit), s, x, tasks, len, blocks, o, status, mailbox, epoch,  \
                                px ? *px : no_peers, (early ? 0u : 1u) | chain_lag() << 8, done);                                                                \
        else                                                                                                                                \
            B200_LAUNCH_ORDERED((sum_rows_tma_kernel<false, RINGS[I].stages, RINGS[I].chunk>), (unsigned)tasks, 32,                         \
                                ring_bytes(RINGS[I].stages, RINGS[I].chunk), s, x, tasks, len, blocks, dst, status,                         \
                                (unsigned long long *)nullptr, 0u, no_peers, 1u, (unsigned long long *)nullptr);                            \
    }
                B200_RING_CASE(0) B200_RING_CASE(1) B200_RING_CASE(2) B200_RING_CASE(3) B200_RING_CASE(4)
#undef B200_RING_CASE
                if (mailbox) {
                    *peer_done = px != nullptr;
                    chain_opened(prev, next, early, x, len, o, nullptr);
                    return cudaGetLastError();
                }
            } else {
                B200_LAUNCH_ORDERED(sum_rows_kernel, (unsigned)((tasks + SUM_WARPS - 1) / SUM_WARPS), 32 * SUM_WARPS, 0, s, x, tasks, len, blocks, dst);
            }
            if (blocks > 1) B200_LAUNCH_ORDERED(sum_combine_kernel, (unsigned)outer, COMBINE_THREADS, 0, s, (const float *)scratch, blocks, o);
            return cudaGetLastError();
        }
        // Few, long columns: the TMA-staged kernel takes the loading off the ordered chains. Many
        // columns already give the plain thread-per-column kernel enough loads in flight. The tile
        // coordinates are 32-bit and the row pitch must be a multiple of 16 bytes.
        const uint64_t groups_per_outer = (inner + 31) / 32;
        if (base16 && inner % 4 == 0 && inner >= 32 && len >= 128 && total < (1ull << 19) && outer * len < 0x7fffffffull &&
            outer * groups_per_outer <= 0x7fffffffull && staged_kernels_ready(device)) {
            CUtensorMap map;
            int *status = reduce_status_word(device);
            const unsigned ctas = (unsigned)(outer * groups_per_outer);
            // PYTORCHES_B200_SUM_COLS=plain keeps the one-warp form (diagnostic, read once).
            static const bool matrix_loads = [] {
                const char *e = getenv("PYTORCHES_B200_SUM_COLS");
                return !(e && e[0] == 'p');
            }();
            // One CTA per SM can afford tall tiles (256 rows, 32 KiB each, 128 KiB in flight), which halve the
            // per-tile bookkeeping of the chain warp; with more column groups than SMs, three CTAs share an SM.
            const bool tall_tiles = ctas <= (unsigned)sm_count(device) && len >= 1024;
            if (matrix_loads && status && make_cols_tensor_map(&map, x, outer * len, inner, tall_tiles ? 256 : 128)) {
                if (tall_tiles)
                    B200_LAUNCH_ORDERED((sum_cols_ldm_kernel<4, 256>), ctas, 64, ldm_smem(4, 256), s, map, len, inner, (uint32_t)groups_per_outer, o, status);
                else
                    B200_LAUNCH_ORDERED((sum_cols_ldm_kernel<4, 128>), ctas, 64, ldm_smem(4, 128), s, map, len, inner, (uint32_t)groups_per_outer, o, status);
                return cudaGetLastError();
            }
            const bool tall = ctas < 2u * (unsigned)sm_count(device) && len >= 1024;
            if (status && make_cols_tensor_map(&map, x, outer * len, inner, tall ? 256 : 128)) {
                if (tall) B200_LAUNCH_ORDERED(sum_cols_tma_kernel<256>, ctas, 32, cols_smem(256), s, map, len, inner, (uint32_t)groups_per_outer, o, status);
                else B200_LAUNCH_ORDERED(sum_cols_tma_kernel<128>, ctas, 32, cols_smem(128), s, map, len, inner, (uint32_t)groups_per_outer, o, status);
                return cudaGetLastError();
            }
        }
        B200_LAUNCH_ORDERED(sum_cols_kernel, (unsigned)((total + 255) / 256), 256, 0, s, x, total, len, inner, o);
        return cudaGetLastError();
    }
    // MAX writes values, ARGMAX positions, MAX_ARGMAX both.
    const bool arg = kind != REDUCE_MAX;
    float *ov = kind == REDUCE_ARGMAX ? nullptr : out_v;
    int64_t *oi = arg ? out_i : nullptr;
    if (inner != 1) {
        B200_LAUNCH_ORDERED(max_cols_kernel, (unsigned)((total + 255) / 256), 256, 0, s, x, total, len, inner, ov, oi, idx_offset);
        return cudaGetLastError();
    }
    MaxPlan m = plan_max(outer, len, sm_count(device));
    if (!base16) m.vec = 1;
    const uint64_t tasks = outer * m.segs;
    unsigned grid = (unsigned)((tasks + (MAX_CTA / m.tpt) - 1) / (MAX_CTA / m.tpt));
    // A single long row: pick the best segment inside the same launch (see max_combiner). The segment
    // positions then live in the mailbox region, not in scratch: scratch goes back to the allocator
    // when this call returns and the next launch may start before this one's combiner has read them.
    MaxFused fused{};
    bool early = false;
    if (outer == 1 && m.tpt == MAX_CTA && m.segs >= 64 && m.segs <= MAILBOX_SLOTS) {
        int *status = reduce_status_word(device);
        uint32_t epoch = 0;
        unsigned long long *done = nullptr;
        unsigned long long *mailbox = status ? mailbox_for(device, s, &epoch, &done) : nullptr;
        if (mailbox) {
            early = may_overlap(prev, x, len, ov, oi);
            fused = MaxFused{mailbox, epoch, ov, oi, idx_offset, status, px ? *px : no_peers, (int)((early ? 0u : 1u) | chain_lag() << 8), done};
            grid += 1;
            *peer_done = px != nullptr;
        }
    }
    if (!fused.mailbox && !ov && spare_v) ov = spare_v;  // the maximum must rest somewhere until the exchange launch reads it
    float *pv = ov;
    int64_t *pi = oi;
    int64_t off1 = idx_offset;
    if (m.segs > 1) {  // pass 1 writes per-segment results (positions within the row) to scratch
        pv = (float *)scratch;
        pi = arg ? (int64_t *)((char *)scratch + ((tasks * 4 + 15) & ~15ull)) : nullptr;
        off1 = 0;
    }
    if (fused.mailbox) pi = arg ? (int64_t *)(fused.mailbox + MAILBOX_SLOTS) : nullptr;
#define B200_MAX_CASE(TPT, VEC)                                                                                                                        \
    if (m.tpt == TPT && m.vec == VEC) {                                                                                                                \
        if (arg) B200_LAUNCH_ORDERED((max_rows_kernel<TPT, VEC, true>), grid, MAX_CTA, 0, s, x, tasks, len, m.segs, m.seg_len, pv, pi, off1, fused);  \
        else B200_LAUNCH_ORDERED((max_rows_kernel<TPT, VEC, false>), grid, MAX_CTA, 0, s, x, tasks, len, m.segs, m.seg_len, pv, pi, off1, fused);     \
    }
    B200_MAX_CASE(32, 1)
    B200_MAX_CASE(32, 4)
    B200_MAX_CASE(256, 1)
    B200_MAX_CASE(256, 4)
#undef B200_MAX_CASE
    if (fused.mailbox) chain_opened(prev, next, early, x, len, ov, oi);
    if (m.segs > 1 && !fused.mailbox) B200_LAUNCH_ORDERED(max_combine_kernel, (unsigned)outer, 256, 0, s, pv, pi, outer, m.segs, ov, oi, idx_offset);
    return cudaGetLastError();
}
}  // namespace

cudaError_t launch_reduce(ReduceKind kind, const float *x, uint64_t outer, uint64_t len, uint64_t inner, float *out_v, int64_t *out_i,
                          int64_t idx_offset, void *scratch, int device, cudaStream_t s, const PeerXchg *px, LaunchChain *chain, float *spare_v) {
    // Across GPUs the maximum travels with its position. A caller that wants the position only passes
    // out_v = null and `spare_v`, a float of its own that nothing else uses: it is written only when
    // the local result has to rest in memory between two launches (an input too short for a combiner CTA).
    const bool position_only = px && kind == REDUCE_MAX_ARGMAX && !out_v && spare_v;
    if (px && (px->world <= 0 || outer != 1 || inner != 1 || kind == REDUCE_ARGMAX || (!out_v && !position_only) ||
               (kind == REDUCE_MAX_ARGMAX && !out_i)))
        return cudaErrorInvalidValue;
    bool peer_done = false;
    LaunchChain before;
    if (chain) {
        before = *chain;
        chain->tail_open = false;  // unless this launch turns out to be one that leaves its tail open
    }
    cudaError_t e = launch_reduce_local(kind, x, outer, len, inner, out_v, out_i, idx_offset, scratch, device, s, px, &peer_done,
                                        chain ? &before : nullptr, chain, position_only ? spare_v : nullptr);
    if (e != cudaSuccess || !px || peer_done) return e;
    if (chain) chain->tail_open = false;
    if (position_only) out_v = spare_v;  // where the local pass left this GPU's maximum
    int *status = reduce_status_word(device);
    if (!status) return cudaErrorMemoryAllocation;
    B200_LAUNCH_ORDERED(peer_exchange_kernel, 1, 32, 0, s, *px, (int)kind, out_v, kind == REDUCE_MAX_ARGMAX ? out_i : (int64_t *)nullptr, status);
    return cudaGetLastError();
}

cudaError_t launch_peer_vector_sum(const PeerXchg &px, const float *partial, uint64_t m, float *out, int device, cudaStream_t s) {
    if (px.world <= 0 || m == 0 || m > PEER_VECTOR_MAX) return cudaErrorInvalidValue;
    int *status = reduce_status_word(device);
    if (!status) return cudaErrorMemoryAllocation;
    B200_LAUNCH_ORDERED(peer_vector_sum_kernel, (unsigned)((m + 255) / 256), 256, 0, s, px, partial, (uint32_t)m, out, status);
    return cudaGetLastError();
}

uint64_t peer_vector_max() { return PEER_VECTOR_MAX; }
uint64_t peer_blocks_max() { return PEER_BLOCKS_MAX; }

cudaError_t launch_argmax_combine(const float *vals, const int64_t *idx, uint64_t g, uint64_t m, int64_t *out, cudaStream_t s) {
    B200_LAUNCH_ORDERED(argmax_combine_kernel, (unsigned)((m + 255) / 256), 256, 0, s, vals, idx, g, m, out);
    return cudaGetLastError();
}

}  // namespace b200

// ---- a sum for callers that must not allocate ------------------------------------------------------------
//
// pytorches_b200_sum_noalloc is the full-tensor SUM_AXIS above with one difference: the per-block
// partial sums that pass 1 hands to pass 2 live in a fixed array inside this library instead of a
// block obtained from the plugin's allocator. It exists for hosts that may not create device memory
// at the moment they need a sum: a process that gave all of the GPU's memory to its own pool at
// start-up (an inference server, another framework's caching allocator), or one under a rule that
// nothing on its hot path may call into the driver's allocator because such a call can stall the
// whole device. Those hosts own the input and output buffers already; the only thing they lacked was
// the scratch, and here it costs no call at all.
//
// The array is 256 KiB of every GPU that loads this library, held until the process exits. It has
// room for 65536 block sums, which bounds the input at 2^32 elements (16 GiB of f32).
namespace b200 {
namespace {

constexpr uint64_t NOALLOC_MAX_BLOCKS = 1ull << 16;
constexpr uint64_t NOALLOC_MAX_ELEMS = NOALLOC_MAX_BLOCKS * SUM_BLOCK;  // 2^32

// Device-side storage. In host code this name is only a handle for cudaGetSymbolAddress, never a
// pointer a kernel could use.
static __device__ __align__(256) float g_noalloc_partials[NOALLOC_MAX_BLOCKS];

std::mutex g_noalloc_mu;
float *g_noalloc_ptr[64] = {};  // per device: the array's address in that device's memory

}  // namespace
}  // namespace b200

extern "C" __attribute__((visibility("default"))) int32_t pytorches_b200_sum_noalloc(uint32_t device, const float *x, uint64_t n,
                                                                                    float *out, void *stream) {
    using namespace b200;
    try {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || (int)device >= count || device >= 64) {
            (void)cudaGetLastError();
            set_last_error("b200: sum_noalloc: no such device");
            return 3;  // PT_STATUS_INVALID_ARGUMENT
        }
        if (n > NOALLOC_MAX_ELEMS) {
            char msg[160];
            std::snprintf(msg, sizeof msg, "b200: sum_noalloc: %llu elements exceed the built-in scratch (at most %llu)",
                          (unsigned long long)n, (unsigned long long)NOALLOC_MAX_ELEMS);
            set_last_error(msg);
            return 3;
        }
        if (!out || (n && !x)) {
            set_last_error("b200: sum_noalloc: null input or output");
            return 3;
        }
        // The caller's current device is put back before returning: a host framework that set it for its
        // own work must not find it changed by a library call.
        struct RestoreDevice {
            int prev = -1;
            ~RestoreDevice() { if (prev >= 0) (void)cudaSetDevice(prev); }
        } restore;
        if (cudaGetDevice(&restore.prev) != cudaSuccess) {
            (void)cudaGetLastError();
            restore.prev = -1;
        }
        if (restore.prev == (int)device) restore.prev = -1;  // nothing to put back
        cudaError_t e = cudaSetDevice((int)device);
        float *partials = nullptr;
        if (e == cudaSuccess) {
            // Once per device, with that device current: ask the runtime where the array lives there.
            std::lock_guard<std::mutex> lock(g_noalloc_mu);
            if (!g_noalloc_ptr[device]) {
                void *p = nullptr;
                e = cudaGetSymbolAddress(&p, g_noalloc_partials);
                if (e == cudaSuccess) g_noalloc_ptr[device] = (float *)p;
            }
            partials = g_noalloc_ptr[device];
        }
        if (e != cudaSuccess) {
            char msg[160];
            std::snprintf(msg, sizeof msg, "b200: sum_noalloc: device set-up failed: %s", cudaGetErrorString(e));
            (void)cudaGetLastError();
            set_last_error(msg);
            return 4;  // PT_STATUS_INTERNAL
        }
        cudaStream_t s = (cudaStream_t)stream;
        note_foreign_enqueue((int)device);  // `stream` may be the plugin's own: what follows there starts the ordinary way
        if (n == 0) {
            e = launch_fill(out, 1, 0.0f, s);  // the sum of nothing is 0.0 (reduce.rs:106-109)
        } else if (n < 32) {
            B200_LAUNCH(sum_short_rows_kernel, 1, 256, 0, s, x, (uint64_t)1, (uint32_t)n, out);
            e = cudaGetLastError();
        } else {
            // Pass 1 overwrites partials[0 .. blocks) completely before pass 2 reads them, so what an
            // earlier call left in the array never matters and nothing needs clearing.
            const uint64_t blocks = (n + SUM_BLOCK - 1) / SUM_BLOCK;
            float *dst = blocks == 1 ? out : partials;
            B200_LAUNCH(sum_rows_kernel, (unsigned)((blocks + SUM_WARPS - 1) / SUM_WARPS), 32 * SUM_WARPS, 0, s, x, blocks, n, blocks, dst);
            if (blocks > 1) B200_LAUNCH(sum_combine_kernel, 1, COMBINE_THREADS, 0, s, (const float *)partials, blocks, out);
            e = cudaGetLastError();
        }
        if (e != cudaSuccess) {
            char msg[160];
            std::snprintf(msg, sizeof msg, "b200: sum_noalloc: launch failed: %s", cudaGetErrorString(e));
            set_last_error(msg);
            return 4;
        }
        return 0;
    } catch (...) {
        set_last_error("b200: sum_noalloc raised an exception");
        return 4;
    }
}

// ---- exercising the expired-wait path without a fault --------------------------------------------------
// A one-warp kernel arms an mbarrier for bytes that no copy will ever deliver, waits for it with a
// small limit, and reports the expiry exactly as the staged reduction kernels would. Nothing hangs and
// nothing faults: the wait simply runs out. Lets a host (and the test suite) check that an expired
// device-side wait surfaces as an error from the next blocking call and that the device stays usable.
namespace b200 {
namespace {
__global__ void __launch_bounds__(32) expired_wait_kernel(int *status, uint32_t limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(&bar, 16);  // nobody sends these 16 bytes
    }
    __syncwarp();
    bool done = false;
    for (uint32_t tries = 0; tries < limit && !done; ++tries) done = mbar_try_wait(&bar, 0);
    if (!done && threadIdx.x == 0) {
        *(volatile int *)status = STATUS_WAIT_EXPIRED;
        __threadfence_system();
    }
}
}  // namespace
}  // namespace b200

extern "C" __attribute__((visibility("default"))) int32_t pytorches_b200_selftest_expired_wait(uint32_t device, void *stream) {
    using namespace b200;
    try {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || (int)device >= count) {
            (void)cudaGetLastError();
            set_last_error("b200: selftest_expired_wait: no such device");
            return 3;
        }
        int *status = reduce_status_word((int)device);
        if (!status || cudaSetDevice((int)device) != cudaSuccess) {
            (void)cudaGetLastError();
            set_last_error("b200: selftest_expired_wait: set-up failed");
            return 4;
        }
        note_foreign_enqueue((int)device);
        B200_LAUNCH(expired_wait_kernel, 1, 32, 0, (cudaStream_t)stream, status, 2000u);
        return cudaGetLastError() == cudaSuccess ? 0 : 4;
    } catch (...) {
        return 4;
    }
}
