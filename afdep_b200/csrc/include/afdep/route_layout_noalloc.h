/* Routing layout without any allocation: an added entry point with no counterpart in the
 * reference library.
 *
 * Who it is for.  `route_layout` (see route_layout_api.h and afdep_b200.ops.route_layout)
 * asks its caller for zero-filled global scratch, and the Python wrapper gets that from
 * torch's allocator on every call.  Some callers cannot do either: code that runs inside a
 * serving engine's pre-planned memory pool and must not grow it, plugins loaded into a
 * process whose allocator they do not own, and hosts written in C that link this library
 * without torch.  For them cudaMalloc (or an allocating library routine) in the middle of a
 * step is either forbidden or a latency spike they cannot afford.
 *
 * What it does.  Same result as `route_layout`: for the [tokens, top_k] int64 expert ids of
 * one source it writes the cleaned ids, the position of each choice among the source's
 * choices of that expert, the record slot of each (token, FFN rank) pair and the totals.
 * The caller passes inputs and outputs only.  The cross-CTA scratch the kernel needs lives
 * in a file-scope __device__ array inside the library, 67,648 bytes, which every GPU that
 * loads the library holds until the process exits.
 *
 * Limits (larger values are rejected with AFDEP_NOALLOC_TOO_LARGE and a message):
 *   num_experts <= 256, ffn_ranks <= 8, top_k <= 32, num_experts % ffn_ranks == 0.
 *
 * Rules of use.
 *   - The first call on a device looks the array's device address up and caches it
 *     (cudaGetSymbolAddress, with that device current).  Make that first call outside any
 *     CUDA stream capture.
 *   - All calls on a device share the one array.  The array keeps what the previous call
 *     left; the kernel tags its entries with a launch counter and the entry point clears
 *     the error words at the start of each call, so nothing else needs resetting — but two
 *     calls that overlap on the GPU (different streams, no ordering between them) race on
 *     it.  Serialise them.
 *   - Nothing here calls cudaMalloc, cudaFree or any routine that allocates.
 *
 *   - The cached address belongs to the device's context at the time of that first call.
 *     After cudaDeviceReset (or any other teardown of that context) the cache is stale:
 *     do not call this entry point again in such a process.
 *
 * What the return value covers, and what it does not.  A return of 0 means the arguments
 * were accepted and the kernel was launched; like any launch, the work itself finishes later
 * on `stream`.  Two outcomes only show in the outputs, after the stream has been synchronised:
 *   - An illegal token (an id outside [-1, num_experts), or an expert named twice) is not an
 *     error code.  All of that token's choices come back as route_e == -1, its tok_slot
 *     entries as -1, and it is left out of the counts; every other token is laid out as
 *     usual.  (The number of such tokens is kept in scratch the caller cannot read: compare
 *     route_e with ids if you need it.)
 *   - If the CTAs' wait on one another runs out of its five-second budget (which needs a GPU
 *     so oversubscribed that the grid is not resident together), every entry of counts[]
 *     comes back as -1 and route_pos / tok_slot hold CTA-local values that must not be used.
 *     A caller that cannot tolerate this checks counts[0] >= 0 before consuming the rest.
 *
 * Returns 0 when the launch was issued, or one of the codes below; the function
 * `afdep_route_layout_noalloc_error` gives the text of the calling thread's last failure.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define AFDEP_NOALLOC_MAX_EXPERTS 256
#define AFDEP_NOALLOC_MAX_FFN_RANKS 8
#define AFDEP_NOALLOC_MAX_TOP_K 32
#define AFDEP_NOALLOC_SCRATCH_BYTES 67648

#define AFDEP_NOALLOC_OK 0
#define AFDEP_NOALLOC_BAD_ARGUMENT 1
#define AFDEP_NOALLOC_TOO_LARGE 2
#define AFDEP_NOALLOC_CUDA_ERROR 3

/* ids:       device, int64 [tokens][top_k]
 * route_e:   device, int32 [tokens][top_k]
 * route_pos: device, int32 [tokens][top_k]
 * tok_slot:  device, int32 [tokens][ffn_ranks]
 * counts:    device, int32 [ffn_ranks + num_experts]
 * stream:    a cudaStream_t (0 for the default stream) */
int afdep_route_layout_noalloc(const long long* ids, int tokens, int top_k, int num_experts, int ffn_ranks,
                               int* route_e, int* route_pos, int* tok_slot, int* counts, void* stream);

const char* afdep_route_layout_noalloc_error(void);

#ifdef __cplusplus
}
#endif
