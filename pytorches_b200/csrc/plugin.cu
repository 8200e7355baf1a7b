// pytorches_plugin_b200: the C-ABI boundary of the B200 backend.
//
// Implements the pytorches plugin vtable (crates/plugin-abi/src/lib.rs:152-191, restated in
// include/pytorches_plugin_abi.h) over the kernels in ew.cu and reduce.cu. It mirrors the behaviour of
// the reference CPU plugin's boundary, plugins/cpu/src/lib.rs: argument validation and status codes
// (lib.rs:250-334), a size-bucketed cache of freed buffers (lib.rs:36-134), and "never unwind across
// the boundary" (lib.rs:345-352). What differs is what a GPU needs:
//   * one in-order CUDA stream per device is the ABI's "implicit default stream"
//     (docs/plugin-abi.md:142-158): execute and host-to-device copies enqueue and return, copy_to_host
//     and synchronize block, and a freed buffer can be handed out again at once because its next use
//     is ordered behind its last one on the same stream (docs/plugin-abi.md:133-135);
//   * the CUDA runtime is linked statically and loads the driver lazily, so loading this library and
//     calling device_count on a machine without a GPU or driver quietly reports zero devices
//     (docs/plugin-abi.md:104-108);
//   * there is no CPU fallback of any kind: without a usable GPU the plugin has no devices.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../../include/pytorches_b200_ext.h"
#include "../../include/pytorches_plugin_abi.h"
#include "common.cuh"

namespace b200 {

std::atomic<uint64_t> g_kernel_launches{0};

namespace {

constexpr int MAX_DEVICES = 16;

thread_local char g_err[512] = "b200: no error";

void set_err(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

struct DeviceState {
    std::mutex mu;                 // serialises calls into one device (docs/plugin-abi.md:232-233)
    bool ready = false;
    cudaStream_t stream = nullptr;
    int sms = 0;
    size_t total_mem = 0;
    std::unordered_map<size_t, std::vector<void *>> free_by_size;  // cached blocks per bucket
    std::unordered_map<void *, size_t> live;                      // handed-out blocks -> bucket
    size_t cached_bytes = 0;
    cudaError_t deferred = cudaSuccess;  // a fault seen after its call had already returned OK
    LaunchChain chain;                   // whether the last thing enqueued leaves room for the next reduction to start early
};

DeviceState g_dev[MAX_DEVICES];
std::once_flag g_count_once;
int g_count = 0;

int visible_devices() {
    std::call_once(g_count_once, [] {
        int n = 0;
        // Fails (without printing) when there is no driver or no GPU: zero devices, not an error.
        if (cudaGetDeviceCount(&n) != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
        g_count = n > MAX_DEVICES ? MAX_DEVICES : n;
    });
    return g_count;
}

// Makes `device` current on the calling thread and sets it up on first use. Call with d.mu held.
cudaError_t ensure_device(uint32_t device) {
    DeviceState &d = g_dev[device];
    cudaError_t e = cudaSetDevice((int)device);
    if (e != cudaSuccess) return e;
    if (d.ready) return cudaSuccess;
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, (int)device)) != cudaSuccess) return e;
    if ((e = cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking)) != cudaSuccess) return e;
    d.sms = prop.multiProcessorCount;
    d.total_mem = prop.totalGlobalMem;
    d.ready = true;
    return cudaSuccess;
}

PtStatus cuda_fail(const char *what, cudaError_t e) {
    set_err("b200: %s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    (void)cudaGetLastError();
    return e == cudaErrorMemoryAllocation ? PT_STATUS_OUT_OF_MEMORY : PT_STATUS_INTERNAL;
}

// ---- memory -------------------------------------------------------------------------------------------------

// Same buckets as the reference (plugins/cpu/src/lib.rs:37-40): powers of two below 1 MiB (at least
// 256 bytes here, the alignment cudaMalloc gives), 2 MiB steps above.
size_t bucket(size_t bytes) {
    constexpr size_t MIB = size_t(1) << 20;
    if (bytes < MIB) {
        size_t p = 256;
        while (p < bytes) p <<= 1;
        return p;
    }
    return (bytes + 2 * MIB - 1) / (2 * MIB) * (2 * MIB);
}

void flush_cache(DeviceState &d) {
    for (auto &kv : d.free_by_size)
        for (void *p : kv.second) (void)cudaFree(p);
    d.free_by_size.clear();
    d.cached_bytes = 0;
}

// Allocation under d.mu with the device current. Reuses a cached block of the same bucket; on
// failure gives the cache back to the driver and retries once (docs/plugin-abi.md:129-130).
PtStatus alloc_locked(DeviceState &d, size_t bytes, void **out) {
    if (bytes > d.total_mem) {  // docs/plugin-abi.md:126-128: fail fast, stay usable
        set_err("b200: alloc of %zu bytes: out of memory (device has %zu bytes)", bytes, d.total_mem);
        return PT_STATUS_OUT_OF_MEMORY;
    }
    const size_t size = bucket(bytes);
    auto it = d.free_by_size.find(size);
    if (it != d.free_by_size.end() && !it->second.empty()) {
        *out = it->second.back();
        it->second.pop_back();
        d.cached_bytes -= size;
        d.live[*out] = size;
        return PT_STATUS_OK;
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, size);
    if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        // Cached blocks may still be in use by queued work: wait for it before returning them.
        (void)cudaStreamSynchronize(d.stream);
        flush_cache(d);
        e = cudaMalloc(&p, size);
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_err("b200: alloc of %zu bytes: cudaMalloc of %zu bytes: %s", bytes, size, cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? PT_STATUS_OUT_OF_MEMORY : PT_STATUS_INTERNAL;
    }
    d.live[p] = size;
    *out = p;
    return PT_STATUS_OK;
}

void free_locked(DeviceState &d, void *ptr) {
    auto it = d.live.find(ptr);
    if (it == d.live.end()) return;  // not ours, or freed twice: ignore rather than corrupt the cache
    const size_t size = it->second;
    d.live.erase(it);
    // Keep at most half of the device cached; beyond that give blocks back. cudaFree waits for the
    // device, so queued work that still uses the block finishes first.
    if (d.cached_bytes + size > d.total_mem / 2) {
        (void)cudaFree(ptr);
        return;
    }
    d.free_by_size[size].push_back(ptr);
    d.cached_bytes += size;
}

bool valid_device(uint32_t device) { return (int)device < visible_devices(); }

#define B200_ENTER(device)                                                    \
    if (!valid_device(device)) {                                              \
        set_err("b200: device %u does not exist", (unsigned)(device));        \
        return PT_STATUS_INVALID_ARGUMENT;                                    \
    }                                                                         \
    DeviceState &d = g_dev[device];                                           \
    std::lock_guard<std::mutex> lock(d.mu);                                   \
    if (cudaError_t e_ = ensure_device(device); e_ != cudaSuccess) return cuda_fail("device setup", e_)

PtStatus alloc_buf(uint32_t device, size_t bytes, void **out) {
    try {
        if (!out) return PT_STATUS_INVALID_ARGUMENT;
        B200_ENTER(device);
        return alloc_locked(d, bytes, out);
    } catch (...) {
        set_err("b200: alloc raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

void free_buf(uint32_t device, void *ptr) {
    try {
        if (!ptr || !valid_device(device)) return;
        DeviceState &d = g_dev[device];
        std::lock_guard<std::mutex> lock(d.mu);
        if (ensure_device(device) != cudaSuccess) return;
        free_locked(d, ptr);
    } catch (...) {
    }
}

// A deferred fault is reported by the next call that can (docs/plugin-abi.md:155-156).
PtStatus finish_blocking(DeviceState &d, const char *what) {
    d.chain.tail_open = false;
    cudaError_t e = cudaStreamSynchronize(d.stream);
    if (e == cudaSuccess) {
        const int gave_up = take_reduce_status((int)(&d - g_dev));
        if (gave_up == 2) {
            set_err("b200: %s: a sharded reduction waited in vain for a peer GPU's result (bounded device-side wait); its result is invalid", what);
            return PT_STATUS_INTERNAL;
        }
        if (gave_up != 0) {
            set_err("b200: %s: a reduction kernel gave up on a bounded device-side wait; its result is invalid", what);
            return PT_STATUS_INTERNAL;
        }
    }
    if (e == cudaSuccess && d.deferred != cudaSuccess) {
        e = d.deferred;
        d.deferred = cudaSuccess;
    }
    return e == cudaSuccess ? PT_STATUS_OK : cuda_fail(what, e);
}

PtStatus copy_from_host(uint32_t device, void *dst, const void *src, size_t bytes) {
    try {
        B200_ENTER(device);
        if (bytes == 0) return PT_STATUS_OK;
        d.chain.tail_open = false;
        cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, d.stream);
        if (e != cudaSuccess) return cuda_fail("copy_from_host", e);
        // The source is only the caller's for the duration of this call. Pageable memory has been
        // staged by the time cudaMemcpyAsync returns; pinned memory is read by the DMA engine later,
        // so wait for it.
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, src) != cudaSuccess) {
            (void)cudaGetLastError();
            return finish_blocking(d, "copy_from_host");
        }
        if (attr.type != cudaMemoryTypeUnregistered) return finish_blocking(d, "copy_from_host");
        return PT_STATUS_OK;
    } catch (...) {
        set_err("b200: copy_from_host raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

PtStatus copy_to_host(uint32_t device, void *dst, const void *src, size_t bytes) {
    try {
        B200_ENTER(device);
        if (bytes) {
            cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, d.stream);
            if (e != cudaSuccess) return cuda_fail("copy_to_host", e);
        }
        return finish_blocking(d, "copy_to_host");
    } catch (...) {
        set_err("b200: copy_to_host raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

PtStatus copy_d2d(uint32_t device, void *dst, const void *src, size_t bytes) {
    try {
        B200_ENTER(device);
        if (bytes == 0) return PT_STATUS_OK;
        d.chain.tail_open = false;
        cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, d.stream);
        return e == cudaSuccess ? PT_STATUS_OK : cuda_fail("copy_device_to_device", e);
    } catch (...) {
        set_err("b200: copy_device_to_device raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

PtStatus synchronize(uint32_t device) {
    try {
        B200_ENTER(device);
        return finish_blocking(d, "synchronize");
    } catch (...) {
        set_err("b200: synchronize raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

// ---- devices ------------------------------------------------------------------------------------------------

uint32_t device_count() {
    try {
        return (uint32_t)visible_devices();
    } catch (...) {
        return 0;
    }
}

PtStatus device_info(uint32_t device, PtDeviceInfo *out) {
    try {
        if (!out) return PT_STATUS_INVALID_ARGUMENT;
        B200_ENTER(device);
        cudaDeviceProp prop;
        cudaError_t e = cudaGetDeviceProperties(&prop, (int)device);
        if (e != cudaSuccess) return cuda_fail("device_info", e);
        std::memset(out, 0, sizeof *out);
        std::snprintf(out->name, sizeof out->name, "%.63s", prop.name);
        out->kind = PT_KIND_CUDA;
        size_t free_b = 0, total_b = 0;
        if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
            out->total_memory = total_b;
            // Cached blocks are reusable, so they count as free (plugins/cpu/src/lib.rs:208-209).
            const size_t f = free_b + d.cached_bytes;
            out->free_memory = f < total_b ? f : total_b;
        } else {
            (void)cudaGetLastError();
            out->total_memory = out->free_memory = PT_MEMORY_UNKNOWN;
        }
        out->flags = 0;
        return PT_STATUS_OK;
    } catch (...) {
        set_err("b200: device_info raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

const char *last_error() { return g_err; }

// ---- execute ------------------------------------------------------------------------------------------------

uint32_t supports_op(uint32_t code) {
    switch (code) {
        case PT_OP_NEG: case PT_OP_EXP: case PT_OP_LOG: case PT_OP_RELU: case PT_OP_TANH: case PT_OP_STEP:
        case PT_OP_ADD: case PT_OP_SUB: case PT_OP_MUL: case PT_OP_DIV:
        case PT_OP_MATMUL: case PT_OP_MATMUL_T: case PT_OP_SUM_AXIS: case PT_OP_MAX_AXIS: case PT_OP_ARGMAX_AXIS:
        case PT_OP_MAX_ARGMAX_AXIS: case PT_OP_ARGMAX_COMBINE:
        case PT_OP_COPY: case PT_OP_FILL: case PT_OP_RAND_NORMAL: case PT_OP_RAND_UNIFORM: case PT_OP_AXPY:
        case PT_OP_RELU_GRAD: case PT_OP_ADD_RELU: case PT_OP_SUB_EXP:
            return 1;
        default:
            return 0;
    }
}

// numel with overflow treated as "too big to be real".
bool numel(const uint64_t *shape, uint32_t nd, uint64_t &n) {
    n = 1;
    for (uint32_t i = 0; i < nd; ++i) {
        if (shape[i] != 0 && n > UINT64_MAX / shape[i]) return false;
        n *= shape[i];
    }
    return true;
}

bool same_shape(const PtTensorDesc &a, const PtTensorDesc &b) {
    if (a.ndim != b.ndim) return false;
    for (uint32_t i = 0; i < a.ndim; ++i)
        if (a.shape[i] != b.shape[i]) return false;
    return true;
}

// Host-side coalescing, the reference's rule (plugins/cpu/src/ew.rs:22-43): drop size-1 dims, merge a
// dim into its outer neighbour when that holds for every operand. Returns false if more than
// MAX_DIMS dims remain.
bool coalesce(const uint64_t *shape, uint32_t nd, const uint64_t *const *strides, int nops, EwProblem &p) {
    p.nd = 0;
    p.n = 1;
    for (uint32_t i = 0; i < nd; ++i) {
        const uint64_t s = shape[i];
        p.n *= s;
        if (s == 1) continue;
        EwDim cur{};
        cur.size = s;
        for (int o = 0; o < nops; ++o) cur.stride[o] = strides[o][i];
        if (p.nd > 0) {
            EwDim &last = p.dim[p.nd - 1];
            bool merge = true;
            for (int o = 0; o < nops; ++o) merge = merge && last.stride[o] == cur.stride[o] * s;
            if (merge) {
                last.size *= s;
                for (int o = 0; o < nops; ++o) last.stride[o] = cur.stride[o];
                continue;
            }
        }
        if (p.nd == MAX_DIMS) return false;
        p.dim[p.nd++] = cur;
    }
    return true;
}

float bits_to_f32(int64_t v) {
    const uint32_t b = (uint32_t)v;
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}

const char *op_name(uint32_t op) {
    switch (op) {
        case PT_OP_NEG: return "NEG"; case PT_OP_EXP: return "EXP"; case PT_OP_LOG: return "LOG";
        case PT_OP_RELU: return "RELU"; case PT_OP_TANH: return "TANH"; case PT_OP_STEP: return "STEP";
        case PT_OP_ADD: return "ADD"; case PT_OP_SUB: return "SUB"; case PT_OP_MUL: return "MUL"; case PT_OP_DIV: return "DIV";
        case PT_OP_MATMUL: return "MATMUL"; case PT_OP_MATMUL_T: return "MATMUL_T"; case PT_OP_SUM_AXIS: return "SUM_AXIS";
        case PT_OP_MAX_AXIS: return "MAX_AXIS"; case PT_OP_ARGMAX_AXIS: return "ARGMAX_AXIS"; case PT_OP_COPY: return "COPY";
        case PT_OP_MAX_ARGMAX_AXIS: return "MAX_ARGMAX_AXIS"; case PT_OP_ARGMAX_COMBINE: return "ARGMAX_COMBINE";
        case PT_OP_FILL: return "FILL"; case PT_OP_RAND_NORMAL: return "RAND_NORMAL"; case PT_OP_RAND_UNIFORM: return "RAND_UNIFORM"; case PT_OP_AXPY: return "AXPY";
        case PT_OP_RELU_GRAD: return "RELU_GRAD"; case PT_OP_ADD_RELU: return "ADD_RELU"; case PT_OP_SUB_EXP: return "SUB_EXP";
        default: return "?";
    }
}

#define B200_INVALID(...)                   \
    do {                                    \
        set_err(__VA_ARGS__);               \
        return PT_STATUS_INVALID_ARGUMENT;  \
    } while (0)

// The two appended ops of a sharded argmax (no counterpart in the reference): MAX_ARGMAX_AXIS has two
// outputs and an index offset in ints[1]; ARGMAX_COMBINE reads i64 positions.
PtStatus run_sharded_argmax(DeviceState &d, uint32_t device, uint32_t op, const PtOpAttrs &attrs, const PtTensorDesc *ins, uint32_t n_in,
                            const PtTensorDesc *outs, uint32_t n_out) {
    cudaError_t e = cudaSuccess;
    if (op == PT_OP_MAX_ARGMAX_AXIS) {
        if (n_in != 1 || n_out != 2) B200_INVALID("b200: MAX_ARGMAX_AXIS takes 1 input and 2 outputs, got %u and %u", n_in, n_out);
        const PtTensorDesc &x = ins[0];
        if (x.dtype != PT_DTYPE_F32 || outs[0].dtype != PT_DTYPE_F32 || outs[1].dtype != PT_DTYPE_I64) {
            set_err("b200: MAX_ARGMAX_AXIS needs an f32 input, an f32 and an i64 output");
            return PT_STATUS_UNSUPPORTED;
        }
        if (attrs.ints[0] < 0 || (uint64_t)attrs.ints[0] >= x.ndim)
            B200_INVALID("b200: MAX_ARGMAX_AXIS: axis %lld out of range for %u dims", (long long)attrs.ints[0], x.ndim);
        const uint32_t axis = (uint32_t)attrs.ints[0];
        uint64_t outer, inner, n0, n1;
        const uint64_t len = x.shape[axis];
        if (!numel(x.shape, axis, outer) || !numel(x.shape + axis + 1, x.ndim - axis - 1, inner) || !numel(outs[0].shape, outs[0].ndim, n0) ||
            !numel(outs[1].shape, outs[1].ndim, n1) || outer * inner != n0 || n0 != n1)
            B200_INVALID("b200: MAX_ARGMAX_AXIS: outputs do not have the reduced shape");
        if (n0 == 0) return PT_STATUS_OK;
        if (len == 0) B200_INVALID("b200: MAX_ARGMAX_AXIS over an empty axis has no value");
        void *scratch = nullptr;
        const size_t sb = reduce_scratch_bytes(REDUCE_MAX_ARGMAX, outer, len, inner, (int)device);
        if (sb) {
            PtStatus st = alloc_locked(d, sb, &scratch);
            if (st != PT_STATUS_OK) return st;
        }
        e = launch_reduce(REDUCE_MAX_ARGMAX, (const float *)x.data, outer, len, inner, (float *)outs[0].data, (int64_t *)outs[1].data,
                          attrs.ints[1], scratch, (int)device, d.stream, nullptr, &d.chain);
        if (scratch) free_locked(d, scratch);
    } else {
        if (n_in != 2 || n_out != 1) B200_INVALID("b200: ARGMAX_COMBINE takes 2 inputs and 1 output, got %u and %u", n_in, n_out);
        if (ins[0].dtype != PT_DTYPE_F32 || ins[1].dtype != PT_DTYPE_I64 || outs[0].dtype != PT_DTYPE_I64) {
            set_err("b200: ARGMAX_COMBINE needs f32 values, i64 positions and an i64 output");
            return PT_STATUS_UNSUPPORTED;
        }
        uint64_t m, mo;
        if (ins[0].ndim < 1 || !same_shape(ins[0], ins[1]) || !numel(ins[0].shape + 1, ins[0].ndim - 1, m) ||
            !numel(outs[0].shape, outs[0].ndim, mo) || m != mo)
            B200_INVALID("b200: ARGMAX_COMBINE: inputs must share a [G, ...] shape and the output drop its first dim");
        if (m == 0) return PT_STATUS_OK;
        if (ins[0].shape[0] == 0) B200_INVALID("b200: ARGMAX_COMBINE of zero candidates has no value");
        d.chain.tail_open = false;
        e = launch_argmax_combine((const float *)ins[0].data, (const int64_t *)ins[1].data, ins[0].shape[0], m, (int64_t *)outs[0].data, d.stream);
    }
    if (e != cudaSuccess) return cuda_fail(op_name(op), e);
    return PT_STATUS_OK;
}

// Validation follows plugins/cpu/src/lib.rs:250-334 check for check.
PtStatus run(DeviceState &d, uint32_t device, uint32_t op, const PtOpAttrs &attrs, const PtTensorDesc *ins, uint32_t n_in,
             const PtTensorDesc *outs, uint32_t n_out) {
    if (n_out != 1) B200_INVALID("b200: op %u: %u outputs, expected 1", op, n_out);
    uint32_t need;
    switch (op) {
        case PT_OP_FILL: case PT_OP_RAND_NORMAL: case PT_OP_RAND_UNIFORM: need = 0; break;
        case PT_OP_NEG: case PT_OP_EXP: case PT_OP_LOG: case PT_OP_RELU: case PT_OP_TANH: case PT_OP_STEP: case PT_OP_COPY:
        case PT_OP_SUM_AXIS: case PT_OP_MAX_AXIS: case PT_OP_ARGMAX_AXIS: need = 1; break;
        case PT_OP_ADD: case PT_OP_SUB: case PT_OP_MUL: case PT_OP_DIV: case PT_OP_MATMUL: case PT_OP_MATMUL_T: case PT_OP_AXPY:
        case PT_OP_RELU_GRAD: case PT_OP_ADD_RELU: case PT_OP_SUB_EXP: need = 2; break;
        default:
            set_err("b200: op %u is not implemented", op);
            return PT_STATUS_UNSUPPORTED;
    }
    if (n_in != need) B200_INVALID("b200: %s: %u inputs, expected %u", op_name(op), n_in, need);
    // The only dtype is f32 (docs/plugin-abi.md:171-172); ARGMAX_AXIS alone writes i64.
    for (uint32_t i = 0; i < n_in; ++i)
        if (ins[i].dtype != PT_DTYPE_F32) {
            set_err("b200: %s: input %u has dtype %u, only f32 is supported", op_name(op), i, ins[i].dtype);
            return PT_STATUS_UNSUPPORTED;
        }
    if (outs[0].dtype != (op == PT_OP_ARGMAX_AXIS ? PT_DTYPE_I64 : PT_DTYPE_F32)) {
        set_err("b200: %s: output dtype %u is not supported", op_name(op), outs[0].dtype);
        return PT_STATUS_UNSUPPORTED;
    }
    const PtTensorDesc &o = outs[0];
    uint64_t n;
    if (!numel(o.shape, o.ndim, n)) B200_INVALID("b200: %s: output element count overflows", op_name(op));
    float *out = (float *)o.data;
    cudaError_t e = cudaSuccess;
    if (op != PT_OP_SUM_AXIS && op != PT_OP_MAX_AXIS && op != PT_OP_ARGMAX_AXIS) d.chain.tail_open = false;
    switch (op) {
        case PT_OP_FILL:
            if (n) e = launch_fill(out, n, bits_to_f32(attrs.ints[0]), d.stream);
            break;
        case PT_OP_RAND_NORMAL:
            if (n) e = launch_randn(out, n, (uint64_t)attrs.ints[0], d.stream);
            break;
        case PT_OP_RAND_UNIFORM:
            if (n) e = launch_rand_uniform(out, n, (uint64_t)attrs.ints[0], bits_to_f32(attrs.ints[1]), bits_to_f32(attrs.ints[2]), (uint64_t)attrs.ints[3], d.stream);
            break;
        case PT_OP_NEG: case PT_OP_EXP: case PT_OP_LOG: case PT_OP_RELU: case PT_OP_TANH: case PT_OP_STEP: case PT_OP_COPY: {
            uint64_t nx;
            if (!numel(ins[0].shape, ins[0].ndim, nx) || nx != n)
                B200_INVALID("b200: %s: input has %llu elements, output %llu", op_name(op), (unsigned long long)nx, (unsigned long long)n);
            if (n == 0) break;
            EwProblem p;
            const uint64_t *st[1] = {ins[0].strides};
            if (!coalesce(ins[0].shape, ins[0].ndim, st, 1, p)) {
                set_err("b200: %s: more than %d non-mergeable dims", op_name(op), MAX_DIMS);
                return PT_STATUS_UNSUPPORTED;
            }
            e = launch_unary(op, (const float *)ins[0].data, out, p, d.stream);
            break;
        }
        case PT_OP_ADD: case PT_OP_SUB: case PT_OP_MUL: case PT_OP_DIV:
        case PT_OP_RELU_GRAD: case PT_OP_ADD_RELU: case PT_OP_SUB_EXP: {
            if (!same_shape(ins[0], o) || !same_shape(ins[1], o)) B200_INVALID("b200: %s: operand shapes differ from the output's", op_name(op));
            if (n == 0) break;
            EwProblem p;
            const uint64_t *st[2] = {ins[0].strides, ins[1].strides};
            if (!coalesce(o.shape, o.ndim, st, 2, p)) {
                set_err("b200: %s: more than %d non-mergeable dims", op_name(op), MAX_DIMS);
                return PT_STATUS_UNSUPPORTED;
            }
            e = launch_binary(op, (const float *)ins[0].data, (const float *)ins[1].data, out, p, d.stream);
            break;
        }
        case PT_OP_AXPY: {
            uint64_t na, nb;
            if (!numel(ins[0].shape, ins[0].ndim, na) || !numel(ins[1].shape, ins[1].ndim, nb) || na != n || nb != n)
                B200_INVALID("b200: AXPY: operands have %llu and %llu elements, output %llu", (unsigned long long)na, (unsigned long long)nb, (unsigned long long)n);
            if (n) e = launch_axpy((const float *)ins[0].data, (const float *)ins[1].data, out, bits_to_f32(attrs.ints[0]), n, d.stream);
            break;
        }
        case PT_OP_MATMUL: case PT_OP_MATMUL_T: {
            const PtTensorDesc &A = ins[0], &B = ins[1];
            if (A.ndim != 2 || B.ndim != 2 || o.ndim != 2) B200_INVALID("b200: %s needs 2-D operands", op_name(op));
            const int64_t flags = op == PT_OP_MATMUL_T ? attrs.ints[0] : 0;
            const bool ta = flags & 1, tb = flags & 2;
            const uint64_t m = ta ? A.shape[1] : A.shape[0], k = ta ? A.shape[0] : A.shape[1];
            const uint64_t kb = tb ? B.shape[1] : B.shape[0], nn = tb ? B.shape[0] : B.shape[1];
            if (k != kb || o.shape[0] != m || o.shape[1] != nn)
                B200_INVALID("b200: %s: [%llu,%llu] x [%llu,%llu] does not give [%llu,%llu]", op_name(op), (unsigned long long)m, (unsigned long long)k,
                             (unsigned long long)kb, (unsigned long long)nn, (unsigned long long)o.shape[0], (unsigned long long)o.shape[1]);
            if (n == 0) break;
            if (((m + 31) / 32) * ((nn + 31) / 32) > 0x7fffffffull)
                B200_INVALID("b200: %s: an output of [%llu,%llu] is more than this kernel's 2^31 - 1 tiles of 32x32", op_name(op),
                             (unsigned long long)m, (unsigned long long)nn);
            const uint64_t ars = ta ? A.strides[1] : A.strides[0], acs = ta ? A.strides[0] : A.strides[1];
            const uint64_t brs = tb ? B.strides[1] : B.strides[0], bcs = tb ? B.strides[0] : B.strides[1];
            e = launch_matmul((const float *)A.data, ars, acs, (const float *)B.data, brs, bcs, out, m, nn, k, d.stream);
            break;
        }
        case PT_OP_SUM_AXIS: case PT_OP_MAX_AXIS: case PT_OP_ARGMAX_AXIS: {
            const PtTensorDesc &x = ins[0];
            if (attrs.ints[0] < 0 || (uint64_t)attrs.ints[0] >= x.ndim)
                B200_INVALID("b200: %s: axis %lld out of range for %u dims", op_name(op), (long long)attrs.ints[0], x.ndim);
            const uint32_t axis = (uint32_t)attrs.ints[0];
            uint64_t outer, inner;
            const uint64_t len = x.shape[axis];
            if (!numel(x.shape, axis, outer) || !numel(x.shape + axis + 1, x.ndim - axis - 1, inner) || outer * inner != n)
                B200_INVALID("b200: %s: output has %llu elements, expected %llu", op_name(op), (unsigned long long)n, (unsigned long long)(outer * inner));
            if (n == 0) break;
            const ReduceKind kind = op == PT_OP_SUM_AXIS ? REDUCE_SUM : op == PT_OP_MAX_AXIS ? REDUCE_MAX : REDUCE_ARGMAX;
            if (kind != REDUCE_SUM && len == 0) B200_INVALID("b200: %s over an empty axis has no value", op_name(op));
            // Two-pass reductions keep their per-block partials in a scratch block from the cache; it
            // goes back right after the launches, the stream orders any reuse behind them.
            void *scratch = nullptr;
            const size_t sb = reduce_scratch_bytes(kind, outer, len, inner, (int)device);
            if (sb) {
                PtStatus st = alloc_locked(d, sb, &scratch);
                if (st != PT_STATUS_OK) return st;
            }
            e = launch_reduce(kind, (const float *)x.data, outer, len, inner, kind == REDUCE_ARGMAX ? nullptr : (float *)o.data,
                              kind == REDUCE_ARGMAX ? (int64_t *)o.data : nullptr, 0, scratch, (int)device, d.stream, nullptr, &d.chain);
            if (scratch) free_locked(d, scratch);
            break;
        }
        default:
            return PT_STATUS_UNSUPPORTED;
    }
    if (e != cudaSuccess) return cuda_fail(op_name(op), e);
    return PT_STATUS_OK;
}

PtStatus execute(uint32_t device, uint32_t op, const PtOpAttrs *attrs, const PtTensorDesc *ins, uint32_t n_in,
                 const PtTensorDesc *outs, uint32_t n_out) {
    try {
        PtOpAttrs a{};
        if (attrs) a = *attrs;
        B200_ENTER(device);
        if (op == PT_OP_MAX_ARGMAX_AXIS || op == PT_OP_ARGMAX_COMBINE) return run_sharded_argmax(d, device, op, a, ins, n_in, outs, n_out);
        return run(d, device, op, a, ins, n_in, outs, n_out);
    } catch (...) {
        set_err("b200: op %u raised an exception", op);
        return PT_STATUS_INTERNAL;
    }
}

// ---- reductions over a tensor that is split across GPUs (extension entry points) ----------------------------

PtStatus peer_export(uint32_t device, void *handle) {
    B200_ENTER(device);
    d.chain.tail_open = false;
    cudaError_t e = peer_window_export((int)device, handle, d.stream);
    return e == cudaSuccess ? PT_STATUS_OK : cuda_fail("peer window export", e);
}

PtStatus peer_attach(uint32_t device, uint32_t rank, uint32_t world, const void *handles, uint32_t wait_ms) {
    if (!handles || world == 0 || world > (uint32_t)PEER_MAX_RANKS || rank >= world)
        B200_INVALID("b200: peer attach: rank %u of %u ranks (at most %d)", rank, world, PEER_MAX_RANKS);
    B200_ENTER(device);
    cudaError_t e = peer_window_attach((int)device, rank, world, handles, wait_ms);
    if (e == cudaErrorInvalidValue) B200_INVALID("b200: peer attach: export this device's window first and pass its handle at index `rank`");
    return e == cudaSuccess ? PT_STATUS_OK : cuda_fail("peer window attach (CUDA IPC)", e);
}

PtStatus peer_trace(uint32_t device, uint64_t *out) {
    if (!out) B200_INVALID("b200: peer trace: null pointer");
    B200_ENTER(device);
    d.chain.tail_open = false;
    cudaError_t e = peer_trace_read((int)device, (unsigned long long *)out, d.stream);
    if (e == cudaErrorInvalidValue) B200_INVALID("b200: peer trace: no window on device %u", device);
    return e == cudaSuccess ? PT_STATUS_OK : cuda_fail("peer trace", e);
}

// kind: 0 sum, 1 max, 2 argmax, 3 mean (the sum divided by `count`, the whole tensor's element count as f32).
PtStatus peer_reduce(uint32_t device, uint32_t kind, const float *x, uint64_t n, int64_t first_index, uint64_t seq, void *out, float count = 0.0f) {
    if (kind > 3) B200_INVALID("b200: peer reduce: kind %u is not 0 (sum), 1 (max), 2 (argmax) or 3 (mean)", kind);
    if (!out || (!x && n)) B200_INVALID("b200: peer reduce: null pointer");
    if ((kind == 1 || kind == 2) && n == 0) B200_INVALID("b200: peer reduce: max/argmax of an empty shard has no value");
    if (kind == 3 && !(count > 0.0f)) B200_INVALID("b200: peer mean: the whole tensor's element count must be positive");
    if (((uintptr_t)x & 3) || ((uintptr_t)out & (kind == 2 ? 7 : 3))) B200_INVALID("b200: peer reduce: x must be 4-byte aligned, out aligned to its type");
    B200_ENTER(device);
    PeerXchg px;
    if (!peer_window_for((int)device, seq, &px)) B200_INVALID("b200: peer reduce: no peer windows attached on device %u", device);
    px.divide_by = kind == 3 ? count : 0.0f;
    const ReduceKind rk = (kind == 0 || kind == 3) ? REDUCE_SUM : kind == 1 ? REDUCE_MAX : REDUCE_MAX_ARGMAX;
    void *scratch = nullptr, *value = nullptr;
    const size_t sb = reduce_scratch_bytes(rk, 1, n, 1, (int)device);
    PtStatus st = PT_STATUS_OK;
    if (sb && (st = alloc_locked(d, sb, &scratch)) != PT_STATUS_OK) return st;
    if (kind == 2 && (st = alloc_locked(d, sizeof(float), &value)) != PT_STATUS_OK) {  // the maximum travels with its position
        if (scratch) free_locked(d, scratch);
        return st;
    }
    cudaError_t e = launch_reduce(rk, x, 1, n, 1, kind == 2 ? nullptr : (float *)out, kind == 2 ? (int64_t *)out : nullptr, first_index,
                                  scratch, (int)device, d.stream, &px, &d.chain, (float *)value);
    if (scratch) free_locked(d, scratch);
    if (value) free_locked(d, value);
    return e == cudaSuccess ? PT_STATUS_OK : cuda_fail("peer reduce", e);
}

// The sum (or mean) of a tensor split over the ranks in whole 65536-element blocks, with the bits of the
// sum over the unsplit tensor: every rank chains ALL block sums in block order (see PeerXchg).
PtStatus peer_sum_unsplit(uint32_t device, const float *x, uint64_t n, uint64_t first_index, uint64_t n_total, uint32_t mean, uint64_t seq, float *out) {
    constexpr uint64_t BLOCK = 65536;
    if (!out || !x) B200_INVALID("b200: peer sum in unsplit order: null pointer");
    if (n == 0 || first_index % BLOCK || first_index + n > n_total || (first_index + n != n_total && n % BLOCK))
        B200_INVALID("b200: peer sum in unsplit order: the shard [%llu, %llu) of %llu elements is not a run of whole 65536-element blocks",
                     (unsigned long long)first_index, (unsigned long long)(first_index + n), (unsigned long long)n_total);
    const uint64_t blocks_total = (n_total + BLOCK - 1) / BLOCK;
    if (blocks_total > peer_blocks_max())
        B200_INVALID("b200: peer sum in unsplit order: %llu blocks, the windows hold %llu", (unsigned long long)blocks_total, (unsigned long long)peer_blocks_max());
    if (((uintptr_t)x & 15) || ((uintptr_t)out & 3)) B200_INVALID("b200: peer sum in unsplit order: x must be 16-byte aligned, out 4-byte aligned");
    B200_ENTER(device);
    PeerXchg px;
    if (!peer_window_for((int)device, seq, &px)) B200_INVALID("b200: peer sum in unsplit order: no peer windows attached on device %u", device);
    px.divide_by = mean ? (float)n_total : 0.0f;
    px.block0 = (uint32_t)(first_index / BLOCK);
    px.blocks_total = (uint32_t)blocks_total;
    cudaError_t e = launch_reduce(REDUCE_SUM, x, 1, n, 1, out, nullptr, 0, nullptr, (int)device, d.stream, &px, &d.chain);
    if (e == cudaErrorInvalidValue) B200_INVALID("b200: peer sum in unsplit order: this shard cannot take the one-launch form");
    return e == cudaSuccess ? PT_STATUS_OK : cuda_fail("peer sum in unsplit order", e);
}

// Sum over the leading dimension of a [rows, m] tensor whose rows are split over the ranks: the local
// SUM_AXIS(0) of this rank's rows, then the exchange and rank-ordered combine of the m partial sums.
PtStatus peer_sum_axis0(uint32_t device, const float *x, uint64_t rows, uint64_t m, uint64_t seq, float *out) {
    if (!out || (!x && rows && m)) B200_INVALID("b200: peer sum_axis0: null pointer");
    if (m == 0 || m > peer_vector_max()) B200_INVALID("b200: peer sum_axis0: %llu columns (1 to %llu are exchanged inside the kernel)",
                                                        (unsigned long long)m, (unsigned long long)peer_vector_max());
    if (((uintptr_t)x & 3) || ((uintptr_t)out & 3)) B200_INVALID("b200: peer sum_axis0: pointers must be 4-byte aligned");
    B200_ENTER(device);
    PeerXchg px;
    if (!peer_window_for((int)device, seq, &px)) B200_INVALID("b200: peer sum_axis0: no peer windows attached on device %u", device);
    void *partial = nullptr, *scratch = nullptr;
    PtStatus st = alloc_locked(d, m * sizeof(float), &partial);
    if (st != PT_STATUS_OK) return st;
    const size_t sb = reduce_scratch_bytes(REDUCE_SUM, 1, rows, m, (int)device);
    if (sb && (st = alloc_locked(d, sb, &scratch)) != PT_STATUS_OK) {
        free_locked(d, partial);
        return st;
    }
    d.chain.tail_open = false;
    cudaError_t e = launch_reduce(REDUCE_SUM, x, 1, rows, m, (float *)partial, nullptr, 0, scratch, (int)device, d.stream);
    if (e == cudaSuccess) e = launch_peer_vector_sum(px, (const float *)partial, m, out, (int)device, d.stream);
    d.chain.tail_open = false;
    if (scratch) free_locked(d, scratch);
    free_locked(d, partial);  // the stream orders any reuse behind the launches
    return e == cudaSuccess ? PT_STATUS_OK : cuda_fail("peer sum_axis0", e);
}

// ---- replay of a recorded call list (extension entry point) --------------------------------------------------

static_assert(sizeof(PtB200Operand) == 152 && sizeof(PtB200Call) == 656, "replay structs are part of the C ABI");

PtStatus replay(uint32_t device, const PtB200Call *calls, uint32_t n_calls, uint32_t repeats, uint64_t first_seq) {
    if (!calls && n_calls) B200_INVALID("b200: replay: null call list");
    int64_t max_slot = -1;
    for (uint32_t i = 0; i < n_calls; ++i) {
        const PtB200Call &c = calls[i];
        if (c.kind > PT_B200_CALL_PEER_REDUCE) B200_INVALID("b200: replay: call %u has unknown kind %u", i, c.kind);
        if (c.n_in > 2 || c.n_out > 2) B200_INVALID("b200: replay: call %u has %u inputs and %u outputs (at most 2 each)", i, c.n_in, c.n_out);
        if (c.kind == PT_B200_CALL_ALLOC || c.kind == PT_B200_CALL_FREE) {
            if (c.ints[1] < 0 || c.ints[1] >= (1 << 20)) B200_INVALID("b200: replay: call %u names slot %lld", i, (long long)c.ints[1]);
            if (c.ints[1] > max_slot) max_slot = c.ints[1];
        }
        for (uint32_t k = 0; k < c.n_in + c.n_out; ++k) {
            const PtB200Operand &a = k < c.n_in ? c.in[k] : c.out[k - c.n_in];
            if (a.ndim > 8) B200_INVALID("b200: replay: call %u has an operand of %u dims (at most 8)", i, a.ndim);
            if (a.slot >= (1 << 20)) B200_INVALID("b200: replay: call %u names slot %d", i, a.slot);
            if (a.slot > max_slot) max_slot = a.slot;
        }
    }
    std::vector<void *> slots((size_t)(max_slot + 1), nullptr);
    auto resolve = [&](const PtB200Operand &a, PtTensorDesc &t) {
        t.data = a.slot >= 0 ? slots[(size_t)a.slot] : a.data;
        t.dtype = a.dtype;
        t.ndim = a.ndim;
        t.shape = a.shape;
        t.strides = a.strides;
    };
    // Newest first, so that the allocator's cache hands the blocks out again in the order of the list:
    // a result buffer is then never the one the call just before it wrote.
    auto drop_all = [&] {
        for (size_t i = slots.size(); i-- > 0;)
            if (slots[i]) {
                free_buf(device, slots[i]);
                slots[i] = nullptr;
            }
    };
    uint64_t seq = first_seq;
    for (uint32_t r = 0; r < repeats; ++r) {
        for (uint32_t i = 0; i < n_calls; ++i) {
            const PtB200Call &c = calls[i];
            PtStatus st = PT_STATUS_OK;
            switch (c.kind) {
                case PT_B200_CALL_ALLOC: {
                    void *&slot = slots[(size_t)c.ints[1]];
                    if (slot) free_buf(device, slot);
                    slot = nullptr;
                    st = alloc_buf(device, (size_t)c.ints[0], &slot);
                    break;
                }
                case PT_B200_CALL_FREE: {
                    void *&slot = slots[(size_t)c.ints[1]];
                    if (slot) free_buf(device, slot);
                    slot = nullptr;
                    break;
                }
                case PT_B200_CALL_EXECUTE: {
                    PtTensorDesc ins[2], outs[2];
                    for (uint32_t k = 0; k < c.n_in; ++k) resolve(c.in[k], ins[k]);
                    for (uint32_t k = 0; k < c.n_out; ++k) resolve(c.out[k], outs[k]);
                    PtOpAttrs attrs;
                    std::memcpy(attrs.ints, c.ints, sizeof attrs.ints);
                    st = execute(device, c.op, &attrs, ins, c.n_in, outs, c.n_out);
                    break;
                }
                default: {  // PT_B200_CALL_PEER_REDUCE
                    if (c.n_in != 1 || c.n_out != 1) {
                        drop_all();
                        B200_INVALID("b200: replay: call %u: a sharded reduction takes 1 input and 1 output", i);
                    }
                    PtTensorDesc x, o;
                    resolve(c.in[0], x);
                    resolve(c.out[0], o);
                    uint64_t n;
                    if (!numel(x.shape, x.ndim, n)) n = 0;
                    if (c.op == 4 || c.op == 5)  // sum / mean in unsplit order
                        st = peer_sum_unsplit(device, (const float *)x.data, n, (uint64_t)c.ints[0], (uint64_t)c.ints[1], c.op == 5, seq++, (float *)o.data);
                    else
                        st = peer_reduce(device, c.op, (const float *)x.data, n, c.ints[0], seq++, o.data, (float)c.ints[1]);
                    break;
                }
            }
            if (st != PT_STATUS_OK) {
                drop_all();
                return st;
            }
        }
        drop_all();  // what the list left allocated dies with the step, as when the host drops its results
    }
    return PT_STATUS_OK;
}

const PtPluginVTable VTABLE = {
    PT_ABI_VERSION, PT_VTABLE_SIZE, 1, "b200",
    device_count, device_info, alloc_buf, free_buf, copy_from_host, copy_to_host, copy_d2d,
    supports_op, execute, synchronize, last_error,
};

}  // namespace

void set_last_error(const char *msg) { set_err("%s", msg); }

void note_foreign_enqueue(int device) {
    if (device < 0 || device >= MAX_DEVICES) return;
    std::lock_guard<std::mutex> lock(g_dev[device].mu);
    g_dev[device].chain.tail_open = false;
}

int sm_count(int device) {
    if (device < 0) (void)cudaGetDevice(&device);
    if (device >= 0 && device < MAX_DEVICES && g_dev[device].sms) return g_dev[device].sms;
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) n = 148;
    return n;
}

}  // namespace b200

#define B200_EXPORT __attribute__((visibility("default")))

extern "C" {

B200_EXPORT const PtPluginVTable *pytorches_plugin_entry(void) { return &b200::VTABLE; }

B200_EXPORT void *pytorches_b200_stream(uint32_t device) {
    try {
        if (!b200::valid_device(device)) return nullptr;
        b200::DeviceState &d = b200::g_dev[device];
        std::lock_guard<std::mutex> lock(d.mu);
        if (b200::ensure_device(device) != cudaSuccess) return nullptr;
        return (void *)d.stream;
    } catch (...) {
        return nullptr;
    }
}

B200_EXPORT uint64_t pytorches_b200_kernel_launches(void) { return b200::g_kernel_launches.load(std::memory_order_relaxed); }

B200_EXPORT int32_t pytorches_b200_peer_export(uint32_t device, void *handle_out) {
    try {
        if (!handle_out) return PT_STATUS_INVALID_ARGUMENT;
        return b200::peer_export(device, handle_out);
    } catch (...) {
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT int32_t pytorches_b200_peer_attach(uint32_t device, uint32_t rank, uint32_t world, const void *handles, uint32_t wait_ms) {
    try {
        return b200::peer_attach(device, rank, world, handles, wait_ms);
    } catch (...) {
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT int32_t pytorches_b200_peer_reduce(uint32_t device, uint32_t kind, const float *x, uint64_t n, int64_t first_index, uint64_t seq,
                                               void *out) {
    try {
        if (kind > 2) {
            b200::set_last_error("b200: peer reduce: kind is not 0 (sum), 1 (max) or 2 (argmax)");
            return PT_STATUS_INVALID_ARGUMENT;
        }
        return b200::peer_reduce(device, kind, x, n, first_index, seq, out);
    } catch (...) {
        b200::set_last_error("b200: peer reduce raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT int32_t pytorches_b200_peer_mean(uint32_t device, const float *x, uint64_t n, uint64_t n_total, uint64_t seq, float *out) {
    try {
        return b200::peer_reduce(device, 3, x, n, 0, seq, out, (float)n_total);
    } catch (...) {
        b200::set_last_error("b200: peer mean raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT int32_t pytorches_b200_peer_trace(uint32_t device, uint64_t *records_out) {
    try {
        return b200::peer_trace(device, records_out);
    } catch (...) {
        b200::set_last_error("b200: peer trace raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT int32_t pytorches_b200_peer_sum_unsplit(uint32_t device, const float *x, uint64_t n, uint64_t first_index, uint64_t n_total, uint32_t mean,
                                                    uint64_t seq, float *out) {
    try {
        return b200::peer_sum_unsplit(device, x, n, first_index, n_total, mean, seq, out);
    } catch (...) {
        b200::set_last_error("b200: peer sum in unsplit order raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT int32_t pytorches_b200_peer_sum_axis0(uint32_t device, const float *x, uint64_t rows, uint64_t cols, uint64_t seq, float *out) {
    try {
        return b200::peer_sum_axis0(device, x, rows, cols, seq, out);
    } catch (...) {
        b200::set_last_error("b200: peer sum_axis0 raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT int32_t pytorches_b200_replay(uint32_t device, const PtB200Call *calls, uint32_t n_calls, uint32_t repeats, uint64_t first_seq) {
    try {
        return b200::replay(device, calls, n_calls, repeats, first_seq);
    } catch (...) {
        b200::set_last_error("b200: replay raised an exception");
        return PT_STATUS_INTERNAL;
    }
}

B200_EXPORT void pytorches_b200_stream_touched(uint32_t device) {
    try {
        b200::note_foreign_enqueue((int)device);
    } catch (...) {
    }
}

}  // extern "C"
