/*
 * C restatement of the pytorches plugin ABI (major version 4).
 *
 * The machine-readable original is the Rust crate crates/plugin-abi/src/lib.rs of
 * tonyt123456/pytorches; the normative prose is docs/plugin-abi.md. Every constant, struct
 * and function-pointer type below cites the line of that crate it mirrors. A plugin is a
 * shared library `pytorches_plugin_<name>.so` exporting ONE symbol,
 * `pytorches_plugin_entry`, that returns a pointer to a static PtPluginVTable
 * (crates/plugin-abi/src/lib.rs:42-44,196).
 *
 * Codes marked "appended" do not exist in the reference crate. They follow its append-only
 * rule (crates/plugin-abi/src/lib.rs:28-30,66; docs/plugin-abi.md:92-96,199-201): new op and
 * dtype numbers, no renumbering, no layout change, ABI_VERSION untouched. A core that does
 * not know them never sends them.
 */
#ifndef PYTORCHES_PLUGIN_ABI_H
#define PYTORCHES_PLUGIN_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* crates/plugin-abi/src/lib.rs:35-44 */
#define PT_ABI_VERSION 4u
#define PT_VTABLE_HEADER_SIZE 8u
#define PT_ENTRY_SYMBOL "pytorches_plugin_entry"
#define PT_FILE_PREFIX "pytorches_plugin_"

/* crates/plugin-abi/src/lib.rs:46-51 */
typedef int32_t PtStatus;
#define PT_STATUS_OK 0
#define PT_STATUS_UNSUPPORTED 1
#define PT_STATUS_OUT_OF_MEMORY 2
#define PT_STATUS_INVALID_ARGUMENT 3
#define PT_STATUS_INTERNAL 4

/* crates/plugin-abi/src/lib.rs:53 */
#define PT_DTYPE_F32 0u
/* appended: 64-bit signed integers, used only for the output of PT_OP_ARGMAX_AXIS. */
#define PT_DTYPE_I64 1u

/* crates/plugin-abi/src/lib.rs:55-61 */
#define PT_KIND_CPU 0u
#define PT_KIND_CUDA 1u
#define PT_KIND_ROCM 2u
#define PT_KIND_XPU 3u
#define PT_KIND_NPU 4u
#define PT_KIND_METAL 5u
#define PT_KIND_OTHER 255u

/* crates/plugin-abi/src/lib.rs:64 */
#define PT_MEMORY_UNKNOWN UINT64_MAX

/* Op codes, crates/plugin-abi/src/lib.rs:67-115. */
enum {
    PT_OP_NEG = 1,
    PT_OP_EXP = 2,
    PT_OP_LOG = 3,
    PT_OP_RELU = 4,
    PT_OP_TANH = 5,
    PT_OP_STEP = 6, /* 1.0 where x > 0 else 0.0 */

    PT_OP_ADD = 100, /* binary: both inputs carry the output's shape, stride 0 = broadcast */
    PT_OP_SUB = 101,
    PT_OP_MUL = 102,
    PT_OP_DIV = 103,

    PT_OP_MATMUL = 200,   /* row-major [m,k] x [k,n] -> [m,n] */
    PT_OP_SUM_AXIS = 201, /* sum over axis ints[0], removing it; contiguous input */
    PT_OP_MATMUL_T = 202, /* optional; ints[0] bit0 = A^T, bit1 = B^T over stored operands */

    /* appended: same (outer, len, inner) contract as SUM_AXIS. Values follow torch CPU
     * amax/argmax: a NaN in a reduced slice wins (and its first position is the argmax),
     * ties resolve to the lowest index. ARGMAX_AXIS writes PT_DTYPE_I64 indices. A zero-length
     * axis is PT_STATUS_INVALID_ARGUMENT (there is no identity to return). */
    PT_OP_MAX_AXIS = 203,
    PT_OP_ARGMAX_AXIS = 204,
    /* appended, for reductions sharded over several devices (one pass over the data, then a combine
     * of per-device results; no counterpart in the reference):
     * MAX_ARGMAX_AXIS: one input; TWO outputs over the same reduced shape, outputs[0] the f32 maxima
     *   (as MAX_AXIS) and outputs[1] the i64 positions (as ARGMAX_AXIS) plus ints[1], the position of
     *   this shard's first row in the unsharded axis. It is the only op with two outputs.
     * ARGMAX_COMBINE: inputs[0] f32 [G, ...] candidate maxima and inputs[1] i64 [G, ...] their
     *   positions, one row per shard; output i64 [...]: per column the position of the best
     *   candidate (NaN wins, then the larger value, then the lower position). */
    PT_OP_MAX_ARGMAX_AXIS = 205,
    PT_OP_ARGMAX_COMBINE = 206,

    PT_OP_COPY = 300, /* materialise a strided / broadcast input contiguously */

    PT_OP_FILL = 400,        /* no inputs; ints[0] = f32 bit pattern */
    PT_OP_RAND_NORMAL = 401, /* no inputs; ints[0] = seed; counter-based Box-Muller, see below */
    /* Appended by this plugin, NOT in the reference: uniform values from the same counter hash, so
     * that benchmark inputs of gigabytes can be generated where they are used. No inputs; ints[0] =
     * seed, ints[1] = f32 bits of `lo`, ints[2] = f32 bits of `scale`, ints[3] = counter of element 0.
     * Element i: h = splitmix64(seed ^ (ints[3] + i) * 0x9E3779B97F4A7C15), u = (h >> 40) / 2^24 in
     * [0,1), out = lo + scale * u (one rounded multiply, then one rounded add). */
    PT_OP_RAND_UNIFORM = 402,

    PT_OP_AXPY = 500, /* optional; out = in0 + alpha*in1, alpha bits in ints[0]; out may alias in0 */

    /* Appended by this plugin, NOT in the reference: optional fused ops, each with a fallback in the
     * host (the core asks supports_op and otherwise issues the two ops it stands for), as AXPY has.
     * The reference names them as its next ABI candidates ("a relu gradient, bias plus activation",
     * docs/plugin-abi.md:285-287; TODO.md:270). Operands follow the binary-op contract: both inputs
     * are described with the output's shape and their own strides (0 = broadcast). Each is DEFINED
     * as its two-op sequence through a contiguous intermediate, bit for bit:
     *   RELU_GRAD: out = MUL(in0, STEP(in1))   the gradient the core builds for relu
     *                                          (crates/core/src/lib.rs:639-643); in0 = g, in1 = x
     *   ADD_RELU:  out = RELU(ADD(in0, in1))   bias plus activation
     *   SUB_EXP:   out = EXP(SUB(in0, in1))    the numerator of a row softmax: exp(x - rowmax) */
    PT_OP_RELU_GRAD = 501,
    PT_OP_ADD_RELU = 502,
    PT_OP_SUB_EXP = 503
};

/*
 * RAND_NORMAL recipe (crates/plugin-abi/src/lib.rs:99-107), for element index i (u64):
 *   h  = splitmix64(seed ^ i * 0x9E3779B97F4A7C15)            (wrapping u64)
 *   u1 = ((h >> 40) + 1) / 16777216.0f   in (0,1]
 *   u2 = (h & 0xFFFFFF)  / 16777216.0f   in [0,1)
 *   out = sqrt(-2 ln u1) * cos(2 pi u2)
 *   splitmix64(x): x += 0x9E3779B97F4A7C15; x = (x ^ x>>30) * 0xBF58476D1CE4E5B9;
 *                  x = (x ^ x>>27) * 0x94D049BB133111EB; return x ^ x>>31
 */

/* crates/plugin-abi/src/lib.rs:118-126; strides are in ELEMENTS. */
typedef struct PtTensorDesc {
    void *data;
    uint32_t dtype;
    uint32_t ndim;
    const uint64_t *shape;
    const uint64_t *strides;
} PtTensorDesc;

/* crates/plugin-abi/src/lib.rs:129-133 */
typedef struct PtOpAttrs {
    int64_t ints[4];
} PtOpAttrs;

/* crates/plugin-abi/src/lib.rs:135-145 */
typedef struct PtDeviceInfo {
    char name[64];
    uint32_t kind;
    uint64_t total_memory;
    uint64_t free_memory;
    uint32_t flags;
} PtDeviceInfo;

/* crates/plugin-abi/src/lib.rs:150 */
#define PT_DEVICE_FLAG_SHARED_HOST_MEMORY (1u << 0)

/* crates/plugin-abi/src/lib.rs:152-191 */
typedef struct PtPluginVTable {
    uint32_t abi_version; /* must stay first  */
    uint32_t struct_size; /* must stay second */
    uint32_t plugin_version;
    const char *name;

    uint32_t (*device_count)(void);
    PtStatus (*device_info)(uint32_t device, PtDeviceInfo *out);

    PtStatus (*alloc)(uint32_t device, size_t bytes, void **out);
    void (*free)(uint32_t device, void *ptr);
    PtStatus (*copy_from_host)(uint32_t device, void *dst, const void *src, size_t bytes);
    PtStatus (*copy_to_host)(uint32_t device, void *dst, const void *src, size_t bytes);
    PtStatus (*copy_device_to_device)(uint32_t device, void *dst, const void *src, size_t bytes);

    uint32_t (*supports_op)(uint32_t op);
    PtStatus (*execute)(uint32_t device, uint32_t op, const PtOpAttrs *attrs,
                        const PtTensorDesc *inputs, uint32_t n_inputs,
                        const PtTensorDesc *outputs, uint32_t n_outputs);
    PtStatus (*synchronize)(uint32_t device);
    const char *(*last_error)(void);
} PtPluginVTable;

/* crates/plugin-abi/src/lib.rs:196 */
typedef const PtPluginVTable *(*PtEntryFn)(void);

/* The one exported symbol of a plugin (crates/plugin-abi/src/lib.rs:42). */
const PtPluginVTable *pytorches_plugin_entry(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

/* Layout on x86-64 / aarch64 LP64, as rustc lays out the #[repr(C)] originals. */
#if defined(__cplusplus)
#define PT_STATIC_ASSERT(c, m) static_assert(c, m)
#else
#define PT_STATIC_ASSERT(c, m) _Static_assert(c, m)
#endif
PT_STATIC_ASSERT(sizeof(PtTensorDesc) == 32, "TensorDesc is 32 bytes");
PT_STATIC_ASSERT(offsetof(PtTensorDesc, dtype) == 8, "TensorDesc.dtype @8");
PT_STATIC_ASSERT(offsetof(PtTensorDesc, ndim) == 12, "TensorDesc.ndim @12");
PT_STATIC_ASSERT(offsetof(PtTensorDesc, shape) == 16, "TensorDesc.shape @16");
PT_STATIC_ASSERT(offsetof(PtTensorDesc, strides) == 24, "TensorDesc.strides @24");
PT_STATIC_ASSERT(sizeof(PtOpAttrs) == 32, "OpAttrs is 32 bytes");
PT_STATIC_ASSERT(sizeof(PtDeviceInfo) == 96, "DeviceInfo is 96 bytes");
PT_STATIC_ASSERT(offsetof(PtDeviceInfo, kind) == 64, "DeviceInfo.kind @64");
PT_STATIC_ASSERT(offsetof(PtDeviceInfo, total_memory) == 72, "DeviceInfo.total_memory @72");
PT_STATIC_ASSERT(offsetof(PtDeviceInfo, free_memory) == 80, "DeviceInfo.free_memory @80");
PT_STATIC_ASSERT(offsetof(PtDeviceInfo, flags) == 88, "DeviceInfo.flags @88");
PT_STATIC_ASSERT(sizeof(PtPluginVTable) == 112, "PluginVTable is 112 bytes");
PT_STATIC_ASSERT(offsetof(PtPluginVTable, name) == 16, "PluginVTable.name @16");
PT_STATIC_ASSERT(offsetof(PtPluginVTable, device_count) == 24, "PluginVTable.device_count @24");
PT_STATIC_ASSERT(offsetof(PtPluginVTable, execute) == 88, "PluginVTable.execute @88");
PT_STATIC_ASSERT(offsetof(PtPluginVTable, last_error) == 104, "PluginVTable.last_error @104");

#define PT_VTABLE_SIZE ((uint32_t)sizeof(PtPluginVTable))

#endif /* PYTORCHES_PLUGIN_ABI_H */
