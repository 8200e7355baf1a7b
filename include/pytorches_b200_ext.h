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

#ifdef __cplusplus
}
#endif

#endif /* PYTORCHES_B200_EXT_H */
