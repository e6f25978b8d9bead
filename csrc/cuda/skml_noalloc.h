// skml_compact_noalloc -- gradient compaction for callers that cannot allocate GPU memory.
//
// This entry point has no counterpart in the reference (a JVM program with no GPU code).
//
// Who needs it: code that runs where cudaMalloc / cudaFree are off limits. Examples are a
// plugin called from inside another framework's stream callback or executor thread, code
// running while a memory pool is frozen (during the capture phase of someone else's
// pipeline or under a fixed memory budget handed out at start-up), and real-time loops
// where the implicit device synchronisation of cudaFree is not acceptable. The regular
// entry point, skml_compact, asks the caller for a `block_counts` scratch buffer, which
// such a caller has no way to create.
//
// What it does: exactly what skml_compact does for the sparse kind. The touched-coordinate
// bitmap and the dense accumulator `g` are turned into the sorted (key, value) list
// value = g[k] + lambda * w[k], entries with |value| <= 1e-8 dropped, `g` and `bitmap`
// cleared; meta[0] receives the count and meta[1] the kind (0 empty, 1 sparse; the dense
// kind is never chosen here). Inputs and outputs are still the caller's buffers.
//
// Where the scratch lives: in a device array compiled into the library
// (SKML_NOALLOC_MAX_BLOCKS + 64 unsigned ints, about 16 KB). Every GPU that loads the
// library holds that array until the process exits.
//
// Limits and rules:
//   * dim <= SKML_NOALLOC_MAX_DIM (536,870,912 coordinates); a larger dim is refused with
//     SKML_NOALLOC_TOO_LARGE and a message on stderr, nothing is launched.
//   * The first call on each device looks up the device address of the built-in array
//     (cudaGetSymbolAddress, with that device current) and remembers it. Make that first
//     call before starting any stream capture on that device.
//   * The function itself calls no cudaMalloc, cudaFree or allocating library routine.
//   * All calls on one device share the one array. A call rewrites every entry it reads,
//     so leftovers of the previous call do no harm; but two calls that overlap on the GPU
//     (different streams, no ordering between them) race on it. Order them.
//   * Returns 0, a negative SKML_NOALLOC_* code, or a cudaError_t value.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define SKML_NOALLOC_MAX_BLOCKS 4096
#define SKML_NOALLOC_MAX_DIM (4096ll * 4096ll * 32ll) /* blocks x bitmap words per block x bits */
#define SKML_NOALLOC_BAD_ARGUMENT (-1)
#define SKML_NOALLOC_TOO_LARGE (-2)

int skml_compact_noalloc(float* g, const float* w, unsigned int* bitmap, int dim, float lambda, long long* meta,
                         int* keys, float* vals, long long capacity, unsigned int* status, void* stream);

#ifdef __cplusplus
}
#endif
