/* Exports that only libhc-gpu-runtime-loader.so has, next to the ol* ABI of
 * offload_api.h. */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Directories searched, in order, for `libhc-<backend>-runtime.so` before the
 * bare library name is tried.  The strings are copied.  `count == 0` clears
 * the list.
 * reference: gpu-runtime/loader/src/Loader.cpp:20-39 */
__attribute__((visibility("default"))) void
setGPULoaderSearchPaths(const char *paths[], size_t count);

/* Nonzero: print "<function> enter" / "<function> exit" to stdout around every
 * ol* call; olLaunchKernel also prints grid, block, argument count and shared
 * memory size.
 * reference: gpu-runtime/loader/src/Loader.cpp:41-45, 48-149 */
__attribute__((visibility("default"))) void enableFuncTracing(int val);

#ifdef __cplusplus
}
#endif
