// TEST INFRASTRUCTURE ONLY.
//
// `pytorches_plugin_cpuref.so`: the CPU oracle. A C++ restatement of the reference CPU plugin's
// boundary (plugins/cpu/src/lib.rs) over the kernels in kernels.hpp, exporting the same vtable
// through `pytorches_plugin_entry`, so the same harness drives the oracle and the B200 plugin.
// The reference itself is Rust and cannot be built where this runs; this file and its headers
// are what parity tests, the smoke check and the benchmark's CPU-baseline leg compare against.
// The shipped plugin never links, loads or calls it.
//
// Pinned against the reference's own vectors: RAND_NORMAL golden values
// (crates/core/src/lib.rs:929-937), the exact small cases of crates/core/src/lib.rs:830-894, and
// every case of plugins/cpu/tests/kernels.rs. Bit-equality with a Rust build is by construction
// (same intrinsics, same order); it could not be checked by running the Rust plugin.
// MAX_AXIS / ARGMAX_AXIS / DTYPE_I64 are not in the reference: parity unpinned there, pinned
// against torch CPU here.
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "../../include/pytorches_plugin_abi.h"
#include "kernels.hpp"

namespace {

using namespace cpuref;

constexpr size_t HEADER = 64;  // lib.rs:31: header size and allocation alignment
thread_local char g_err[256] = "cpuref: no error";

void set_err(const char *fmt, unsigned long long a = 0, unsigned long long b = 0) {
    std::snprintf(g_err, sizeof g_err, fmt, a, b);
}

// ---- memory (lib.rs:36-134): size-bucketed cache of freed buffers --------------------------------

size_t bucket(size_t bytes) {  // lib.rs:37-40
    constexpr size_t MIB = size_t(1) << 20;
    if (bytes < MIB) {
        size_t b = std::max(bytes, (size_t)64), p = 1;
        while (p < b) p <<= 1;
        return p;
    }
    return (bytes + 2 * MIB - 1) / (2 * MIB) * (2 * MIB);
}

std::mutex g_cache_mu;
std::unordered_map<size_t, std::vector<void *>> g_cache;
size_t g_cached_bytes = 0;
constexpr size_t CACHE_CAP = size_t(4) << 30;  // lib.rs:52-58 (min(total/8, 4 GiB); fixed here)

void release_block(void *payload) { std::free((char *)payload - HEADER); }

void *fresh_block(size_t size) {
    void *base = nullptr;
    if (posix_memalign(&base, HEADER, size + HEADER) != 0) return nullptr;
    *(size_t *)base = size;
    return (char *)base + HEADER;
}

void flush_cache_locked() {
    for (auto &kv : g_cache)
        for (void *p : kv.second) release_block(p);
    g_cache.clear();
    g_cached_bytes = 0;
}

PtStatus alloc_buf(uint32_t, size_t bytes, void **out) {
    if (bytes > (size_t(1) << 46)) {  // lib.rs:96: sizes that overflow the layout fail fast
        set_err("alloc of %llu bytes: out of memory", bytes);
        return PT_STATUS_OUT_OF_MEMORY;
    }
    const size_t size = bucket(bytes);
    std::lock_guard<std::mutex> g(g_cache_mu);
    auto it = g_cache.find(size);
    if (it != g_cache.end() && !it->second.empty()) {
        *out = it->second.back();
        it->second.pop_back();
        g_cached_bytes -= size;
        return PT_STATUS_OK;
    }
    void *p = fresh_block(size);
    if (!p) {
        flush_cache_locked();  // lib.rs:107-115: give the cache back and retry once
        p = fresh_block(size);
        if (!p) {
            set_err("alloc of %llu bytes: out of memory", bytes);
            return PT_STATUS_OUT_OF_MEMORY;
        }
    }
    *out = p;
    return PT_STATUS_OK;
}

void free_buf(uint32_t, void *ptr) {
    if (!ptr) return;
    const size_t size = *(size_t *)((char *)ptr - HEADER);
    std::lock_guard<std::mutex> g(g_cache_mu);
    if (g_cached_bytes + size > CACHE_CAP) return release_block(ptr);
    g_cache[size].push_back(ptr);
    g_cached_bytes += size;
}

PtStatus copy_any(uint32_t, void *dst, const void *src, size_t bytes) {
    std::memcpy(dst, src, bytes);
    return PT_STATUS_OK;
}

// ---- device info (lib.rs:153-216) ----------------------------------------------------------------

uint32_t device_count() { return 1; }

PtStatus device_info(uint32_t device, PtDeviceInfo *out) {
    if (device != 0 || !out) return PT_STATUS_INVALID_ARGUMENT;
    std::memset(out, 0, sizeof *out);
    std::snprintf(out->name, sizeof out->name, "cpuref");
    out->kind = PT_KIND_CPU;
    out->total_memory = PT_MEMORY_UNKNOWN;
    out->free_memory = PT_MEMORY_UNKNOWN;
    return PT_STATUS_OK;
}

PtStatus synchronize(uint32_t) { return PT_STATUS_OK; }
const char *last_error() { return g_err; }

// ---- dispatch (lib.rs:228-353) -------------------------------------------------------------------

uint32_t supports_op(uint32_t code) {
    switch (code) {
        case OP_NEG: case OP_EXP: case OP_LOG: case OP_RELU: case OP_TANH: case OP_STEP:
        case OP_ADD: case OP_SUB: case OP_MUL: case OP_DIV:
        case OP_MATMUL: case OP_MATMUL_T: case OP_AXPY: case OP_SUM_AXIS: case OP_COPY: case OP_FILL: case OP_RAND_NORMAL: case OP_RAND_UNIFORM:
        case OP_MAX_AXIS: case OP_ARGMAX_AXIS: case OP_MAX_ARGMAX_AXIS: case OP_ARGMAX_COMBINE:
        case OP_RELU_GRAD: case OP_ADD_RELU: case OP_SUB_EXP:
            return 1;
        default: return 0;
    }
}

size_t numel(const uint64_t *shape, size_t nd) {
    size_t n = 1;
    for (size_t d = 0; d < nd; ++d) n *= (size_t)shape[d];
    return n;
}

bool same_shape(const PtTensorDesc &a, const PtTensorDesc &b) {
    if (a.ndim != b.ndim) return false;
    for (uint32_t d = 0; d < a.ndim; ++d)
        if (a.shape[d] != b.shape[d]) return false;
    return true;
}

// The two appended ops for sharded argmax (not in the reference).
PtStatus run_sharded_argmax(uint32_t op, const PtOpAttrs &attrs, const PtTensorDesc *ins, uint32_t n_in, const PtTensorDesc *outs, uint32_t n_out) {
    if (op == OP_MAX_ARGMAX_AXIS) {
        if (n_in != 1 || n_out != 2) return PT_STATUS_INVALID_ARGUMENT;
        const PtTensorDesc &x = ins[0];
        if (x.dtype != PT_DTYPE_F32 || outs[0].dtype != PT_DTYPE_F32 || outs[1].dtype != PT_DTYPE_I64) return PT_STATUS_UNSUPPORTED;
        if (attrs.ints[0] < 0 || (uint64_t)attrs.ints[0] >= x.ndim) return PT_STATUS_INVALID_ARGUMENT;
        const size_t axis = (size_t)attrs.ints[0];
        const size_t outer = numel(x.shape, axis), len = (size_t)x.shape[axis], inner = numel(x.shape + axis + 1, x.ndim - axis - 1);
        if (outer * inner != numel(outs[0].shape, outs[0].ndim) || outer * inner != numel(outs[1].shape, outs[1].ndim)) return PT_STATUS_INVALID_ARGUMENT;
        if (outer * inner == 0) return PT_STATUS_OK;
        if (len == 0) return PT_STATUS_INVALID_ARGUMENT;
        max_axis((const float *)x.data, outer, len, inner, (float *)outs[0].data, (int64_t *)outs[1].data, attrs.ints[1]);
        return PT_STATUS_OK;
    }
    if (n_in != 2 || n_out != 1) return PT_STATUS_INVALID_ARGUMENT;
    if (ins[0].dtype != PT_DTYPE_F32 || ins[1].dtype != PT_DTYPE_I64 || outs[0].dtype != PT_DTYPE_I64) return PT_STATUS_UNSUPPORTED;
    if (ins[0].ndim < 1 || !same_shape(ins[0], ins[1])) return PT_STATUS_INVALID_ARGUMENT;
    const size_t g = (size_t)ins[0].shape[0], m = numel(ins[0].shape + 1, ins[0].ndim - 1);
    if (m != numel(outs[0].shape, outs[0].ndim)) return PT_STATUS_INVALID_ARGUMENT;
    if (m == 0) return PT_STATUS_OK;
    if (g == 0) return PT_STATUS_INVALID_ARGUMENT;
    argmax_combine((const float *)ins[0].data, (const int64_t *)ins[1].data, g, m, (int64_t *)outs[0].data);
    return PT_STATUS_OK;
}

PtStatus run(uint32_t op, const PtOpAttrs &attrs, const PtTensorDesc *ins, uint32_t n_in, const PtTensorDesc *outs, uint32_t n_out) {
    if (n_out != 1) return PT_STATUS_INVALID_ARGUMENT;  // lib.rs:252-254
    uint32_t need;
    switch (op) {  // lib.rs:255-260
        case OP_FILL: case OP_RAND_NORMAL: case OP_RAND_UNIFORM: need = 0; break;
        case OP_NEG: case OP_EXP: case OP_LOG: case OP_RELU: case OP_TANH: case OP_STEP: case OP_COPY:
        case OP_SUM_AXIS: case OP_MAX_AXIS: case OP_ARGMAX_AXIS: need = 1; break;
        case OP_ADD: case OP_SUB: case OP_MUL: case OP_DIV: case OP_MATMUL: case OP_MATMUL_T: case OP_AXPY:
        case OP_RELU_GRAD: case OP_ADD_RELU: case OP_SUB_EXP: need = 2; break;
        default: return PT_STATUS_UNSUPPORTED;
    }
    if (n_in != need) return PT_STATUS_INVALID_ARGUMENT;
    const PtTensorDesc &o = outs[0];
    const size_t n = numel(o.shape, o.ndim);
    float *out = (float *)o.data;
    switch (op) {
        case OP_FILL: {
            uint32_t bits = (uint32_t)attrs.ints[0];
            float v;
            std::memcpy(&v, &bits, 4);
            fill(out, n, v);
            break;
        }
        case OP_RAND_NORMAL: randn(out, n, (uint64_t)attrs.ints[0]); break;
        case OP_RAND_UNIFORM: {
            uint32_t b1 = (uint32_t)attrs.ints[1], b2 = (uint32_t)attrs.ints[2];
            float lo, scale;
            std::memcpy(&lo, &b1, 4);
            std::memcpy(&scale, &b2, 4);
            rand_uniform(out, n, (uint64_t)attrs.ints[0], lo, scale, (uint64_t)attrs.ints[3]);
            break;
        }
        case OP_NEG: case OP_EXP: case OP_LOG: case OP_RELU: case OP_TANH: case OP_STEP: case OP_COPY:
            if (numel(ins[0].shape, ins[0].ndim) != n) return PT_STATUS_INVALID_ARGUMENT;
            unary(op, (const float *)ins[0].data, ins[0].shape, ins[0].strides, ins[0].ndim, out);
            break;
        case OP_ADD: case OP_SUB: case OP_MUL: case OP_DIV:
            if (!same_shape(ins[0], o) || !same_shape(ins[1], o)) return PT_STATUS_INVALID_ARGUMENT;
            binary(op, (const float *)ins[0].data, ins[0].strides, (const float *)ins[1].data, ins[1].strides, o.shape, o.ndim, out);
            break;
        case OP_RELU_GRAD: case OP_ADD_RELU: case OP_SUB_EXP: {
            // The appended fused ops are DEFINED as the two reference ops they stand for, run one after
            // the other through a contiguous intermediate; here they are computed exactly that way.
            if (!same_shape(ins[0], o) || !same_shape(ins[1], o)) return PT_STATUS_INVALID_ARGUMENT;
            if (n == 0) break;
            std::vector<float> mid(n);
            std::vector<uint64_t> dense(o.ndim ? o.ndim : 1, 1);
            for (size_t d = o.ndim; d-- > 1;) dense[d - 1] = dense[d] * o.shape[d];
            const float *a = (const float *)ins[0].data, *b = (const float *)ins[1].data;
            if (op == OP_RELU_GRAD) {  // MUL(g, STEP(x)), crates/core/src/lib.rs:639-643
                unary(OP_STEP, b, o.shape, ins[1].strides, o.ndim, mid.data());
                binary(OP_MUL, a, ins[0].strides, mid.data(), dense.data(), o.shape, o.ndim, out);
            } else {
                binary(op == OP_ADD_RELU ? OP_ADD : OP_SUB, a, ins[0].strides, b, ins[1].strides, o.shape, o.ndim, mid.data());
                unary(op == OP_ADD_RELU ? OP_RELU : OP_EXP, mid.data(), o.shape, dense.data(), o.ndim, out);
            }
            break;
        }
        case OP_AXPY: {
            if (numel(ins[0].shape, ins[0].ndim) != n || numel(ins[1].shape, ins[1].ndim) != n) return PT_STATUS_INVALID_ARGUMENT;
            uint32_t bits = (uint32_t)attrs.ints[0];
            float alpha;
            std::memcpy(&alpha, &bits, 4);
            axpy((const float *)ins[0].data, (const float *)ins[1].data, out, alpha, n);
            break;
        }
        case OP_MATMUL: case OP_MATMUL_T: {  // lib.rs:291-315
            const PtTensorDesc &A = ins[0], &B = ins[1];
            if (A.ndim != 2 || B.ndim != 2 || o.ndim != 2) return PT_STATUS_INVALID_ARGUMENT;
            const int64_t flags = op == OP_MATMUL_T ? attrs.ints[0] : 0;
            const bool ta = flags & 1, tb = flags & 2;
            const size_t m = ta ? A.shape[1] : A.shape[0], k = ta ? A.shape[0] : A.shape[1];
            const size_t kb = tb ? B.shape[1] : B.shape[0], nn = tb ? B.shape[0] : B.shape[1];
            if (k != kb || o.shape[0] != m || o.shape[1] != nn) return PT_STATUS_INVALID_ARGUMENT;
            const size_t ars = ta ? A.strides[1] : A.strides[0], acs = ta ? A.strides[0] : A.strides[1];
            const size_t brs = tb ? B.strides[1] : B.strides[0], bcs = tb ? B.strides[0] : B.strides[1];
            matmul(m, nn, k, (const float *)A.data, ars, acs, (const float *)B.data, brs, bcs, out);
            break;
        }
        case OP_SUM_AXIS: case OP_MAX_AXIS: case OP_ARGMAX_AXIS: {  // lib.rs:316-329
            const PtTensorDesc &x = ins[0];
            if (attrs.ints[0] < 0 || (uint64_t)attrs.ints[0] >= x.ndim) return PT_STATUS_INVALID_ARGUMENT;
            const size_t axis = (size_t)attrs.ints[0];
            const size_t outer = numel(x.shape, axis), len = (size_t)x.shape[axis];
            const size_t inner = numel(x.shape + axis + 1, x.ndim - axis - 1);
            if (outer * inner != n) return PT_STATUS_INVALID_ARGUMENT;
            if (op == OP_SUM_AXIS) {
                sum_axis((const float *)x.data, outer, len, inner, out);
            } else {
                if (len == 0 && n != 0) return PT_STATUS_INVALID_ARGUMENT;
                if (op == OP_MAX_AXIS) max_axis((const float *)x.data, outer, len, inner, out, nullptr);
                else max_axis((const float *)x.data, outer, len, inner, nullptr, (int64_t *)o.data);
            }
            break;
        }
        default: return PT_STATUS_UNSUPPORTED;
    }
    return PT_STATUS_OK;
}

PtStatus execute(uint32_t, uint32_t op, const PtOpAttrs *attrs, const PtTensorDesc *ins, uint32_t n_in,
                 const PtTensorDesc *outs, uint32_t n_out) {
    try {  // lib.rs:345-352: nothing may unwind across the boundary
        PtOpAttrs a{};
        if (attrs) a = *attrs;
        if (op == OP_MAX_ARGMAX_AXIS || op == OP_ARGMAX_COMBINE) {
            PtStatus s = run_sharded_argmax(op, a, ins, n_in, outs, n_out);
            if (s != PT_STATUS_OK) set_err("cpuref: op %llu failed with status %llu", op, (unsigned long long)s);
            return s;
        }
        // The only dtype is f32 (docs/plugin-abi.md:171-172), except ARGMAX_AXIS's i64 output.
        for (uint32_t i = 0; i < n_in; ++i)
            if (ins[i].dtype != PT_DTYPE_F32) return PT_STATUS_UNSUPPORTED;
        for (uint32_t i = 0; i < n_out; ++i)
            if (outs[i].dtype != (op == OP_ARGMAX_AXIS ? PT_DTYPE_I64 : PT_DTYPE_F32)) return PT_STATUS_UNSUPPORTED;
        PtStatus s = run(op, a, ins, n_in, outs, n_out);
        if (s != PT_STATUS_OK) set_err("cpuref: op %llu failed with status %llu", op, (unsigned long long)s);
        return s;
    } catch (...) {
        set_err("cpuref: op %llu raised an exception", op);
        return PT_STATUS_INTERNAL;
    }
}

const PtPluginVTable VTABLE = {
    PT_ABI_VERSION, PT_VTABLE_SIZE, 1, "cpuref",
    device_count, device_info, alloc_buf, free_buf, copy_any, copy_any, copy_any,
    supports_op, execute, synchronize, last_error,
};

}  // namespace

extern "C" const PtPluginVTable *pytorches_plugin_entry(void) { return &VTABLE; }

// Extra symbol for tests: which code paths this host takes (AVX2+FMA decides the bits of
// exp/log/tanh/axpy/sum), and how many pool threads are in use.
extern "C" int cpuref_has_avx2(void) { return cpuref::has_avx2() ? 1 : 0; }
extern "C" unsigned cpuref_threads(void) { return (unsigned)cpuref::Pool::get().threads(); }
