/* C ABI of libcolabfold_cuda_kernels.so (B200, sm_100a): the AF3-family diffusion sampler.
 *
 * Plain pointers and sizes only. Every entry point either enqueues the CUDA kernel or returns an
 * error; there is no CPU path. Each declaration cites the interface of the reference library
 * (mirditalab/colabfold-cuda-kernels) that it replaces, by file:line inside that project.
 */
#ifndef CCK_B200_H
#define CCK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CCK_NUM_INPUTS 74

/* Error codes of cck_mk_sample. cck_last_error() gives the message of the calling thread's last
 * failure. */
enum {
    CCK_OK = 0,
    CCK_E_ARITY = 1,     /* "MkSample: wrong number of inputs"   (src/diffusion/host.cuh:508-510) */
    CCK_E_WORKSPACE = 2, /* "MkSample: workspace too small"      (src/diffusion/host.cuh:527-529) */
    CCK_E_SHAPE = 3,     /* byte sizes that do not describe one supported model */
    CCK_E_FLAGS = 4,     /* a variant flag bit that this library does not build */
    CCK_E_LAUNCH = 5,    /* CUDA error while enqueueing           (src/diffusion/host.cuh:532-536) */
    CCK_E_DEVICE = 6     /* not an sm_100 device */
};

/* The operator core: what the XLA FFI handler `MkSample` does after unpacking its call frame
 * (src/diffusion/host.cuh:505-538: mk_sample). Enqueues one whole sampling run (every step of
 * every sample) on `stream` and returns without synchronising. Nothing is allocated or freed; all
 * buffers are device memory owned by the caller.
 *   stream      cudaStream_t
 *   ext         device int32[5] {N, NS, exact, seed_lo, seed_hi}, read on the device
 *   in, bytes   the 74 inputs in the operator's order (src/diffusion/dims.cuh:61-74) and their sizes
 *   out         f32 [samples][out_tokens][24][3]
 *   ws          workspace of at least mk_workspace_bytes(...) bytes, may be uninitialised
 *   flags       variant bits (src/diffusion/dims.cuh:46-57: bits 0-9). Bits 16-23 are set aside for
 *               variants that only this library has (none is built). A bit that is known but not
 *               built, or a bit outside both ranges, is refused with CCK_E_FLAGS.
 * The first 16 bytes of ws are four control words {barrier, status, where, pad}, cleared by a memset
 * that the call enqueues ahead of the kernel. Every wait inside the kernel is bounded (about a
 * second): a wait that gives up writes status (1 a grid barrier, 2 a wait inside a phase) and where
 * (grid barriers passed), the launch ends at once, normally, and out is filled with NaN instead of
 * coordinates. The reference's waits are unbounded and it has no such words.
 */
int cck_mk_sample(void* stream, const int* ext, const void* const* in, const size_t* bytes, int num_inputs, float* out,
                  int out_tokens, void* ws, size_t ws_bytes, int samples, int nsteps, int flags);
const char* cck_last_error(void);

/* The operator for callers that cannot supply a workspace. It has no counterpart in the reference,
 * which always takes its scratch from the caller. XLA runs the operator on its stream, often while
 * recording a command buffer (CUDA graph), and a C caller may be inside a capture of its own:
 * cudaMalloc is refused there, so such a caller has no way to make scratch. This variant uses a
 * fixed 32 MiB scratch array that the library keeps in device memory on every GPU that loads it.
 * Arguments and result are those of cck_mk_sample without ws / ws_bytes. It allocates nothing.
 *  - A fold whose scratch exceeds cck_static_workspace_bytes() is refused with CCK_E_WORKSPACE
 *    (the message names both sizes): small folds only, e.g. 32 tokens x 1 sample.
 *  - The first call on a device looks up the array's device address; make it outside any capture.
 *  - All calls on a device share the array. Calls ordered on a stream are independent (the control
 *    words are cleared at the start of each call, everything else is written before it is read);
 *    calls that overlap on the GPU race on it and must be ordered by the caller. */
int cck_mk_sample_static(void* stream, const int* ext, const void* const* in, const size_t* bytes, int num_inputs,
                         float* out, int out_tokens, int samples, int nsteps, int flags);
size_t cck_static_workspace_bytes(void);

/* Workspace size for a shape bucket; 0 if the sizes do not describe a supported model
 * (src/diffusion/host.cuh:376-379). */
size_t mk_workspace_bytes(int S, int Nb, int NSb, int nsteps, int flags, const size_t* bytes);

/* Stand-alone debug API, same signatures and meaning as the reference's ctypes API
 * (src/diffusion/host.cuh:381-499, src/diffusion/diffusion.cu:8-31). One global state, not
 * re-entrant. All return 0 on success and 1 on failure unless noted. */
int mk_setup(int S, int N, int A, int NS, int steps, const void** host, const size_t* bytes);
/* mode 0: sample nsteps steps; mode 1: one denoiser call on host xn at level t, result in OUT.
 * dbg_stop > 0 stops after that many phases of the reference's schedule. ms: event-timed launch. */
int mk_run(int mode, int nsteps, int dbg_stop, uint64_t seed, const float* xn, float t, float* ms,
           unsigned long long* timing);
int mk_read(int id, void* host, size_t bytes);
int mk_buf_id(const char* name);  /* -1 if unknown */
size_t mk_buf_bytes(int id);
/* Real extents (tokens, subsets) of the next mk_run calls inside the bucket of mk_setup, as the
 * operator gets them through ext (src/diffusion/host.cuh:219-235); 0, 0 = the bucket's. Scratch
 * buffers are then filled compactly for the real extents. No counterpart in the reference's debug API. */
int mk_set_extent(int N, int NS);
/* The phase program the host writes for the kernel (this implementation's form of the reference's
 * schedule, src/diffusion/sampler.cuh:87-230): up to max_ops operations as 4 bytes each {function,
 * argument, block, end | kind << 2}; returns the program's length or -1. Needs no device. Bit 30 of
 * flags (not an operator flag) asks for the form on completion counters that mk_set_flow(1) runs.
 * No counterpart in the reference's debug API. */
int mk_program(int mode, int nsteps, int flags, unsigned char* ops, int max_ops);
/* 1 (default): a token block runs as one phase (QKVG -> attention -> WO -> adaLN -> W1 -> W2 -> the next
 * block's adaLN), a unit waiting for completion counters of the units it reads; 0: every operation
 * ends at a grid barrier as in the reference's schedule (src/diffusion/sampler.cuh:99-134), which the
 * per-kind timing record and dbg_stop count (mk_run with dbg_stop > 0 always runs on barriers). Same
 * results either way. Returns the previous setting. No counterpart in the reference's debug API. */
int mk_set_flow(int on);
int mk_set_grid(int grid);        /* the grid is one CTA per SM; returns it */
/* The phase kinds of mk_run's timing record, comma-separated. The record (mk_run's `timing`, may be
 * null) is two 64-bit words per kind in this order: wall nanoseconds from grid barrier to grid
 * barrier summed over the kind's phases, and the number of phases. */
const char* mk_timing_names(void);
int mk_version(void);             /* 2: atom adaLN modulations and atom pair logits are f32 */
void mk_teardown(void);
/* C[M][N] (f32) = A[M][K] · W[N][K]^T, bf16 bits in; tile 64/128/256 picks the column tile */
int mk_gemm_test(const uint16_t* A, const uint16_t* W, float* C, int M, int N, int K, int tile);

/* Test doors (no counterpart in the reference). None of them faults or hangs anything: what they
 * provoke is a wait running into its limit, after which the kernel ends normally.
 *  mk_set_attn_skew   the token attention's second pipeline starts `cycles` SM cycles after the first in
 *                     the following runs (0: off). Results must not depend on it. Returns the old value.
 *  mk_set_wait_test   the following runs use `cycles` SM cycles as the limit of every wait (0: the
 *                     default) and their grid barriers expect `extra` arrivals that nobody makes, so
 *                     that with extra > 0 the first barrier gives up: mk_run returns 1, status is 1,
 *                     OUT is NaN. (0, 0) restores production.
 *  mk_wait_test       one thread waits `cycles` SM cycles on an mbarrier that nothing arrives at;
 *                     returns the status the kernel left (2, as it must) or -1 on a CUDA error.
 *  mk_philox_test     the sampler's Philox4x32-10 words (4) and Box-Muller normals (4) for counter
 *                     (idx, step, sample, stream) and key seed, computed on the device
 *                     (src/diffusion/rng.cuh:14-46). */
int mk_set_attn_skew(int cycles);
int mk_set_wait_test(long long cycles, int extra);
int mk_wait_test(long long cycles, float* ms);
int mk_philox_test(uint32_t idx, uint32_t step, uint32_t sample, uint32_t stream, uint64_t seed, uint32_t* words, float* z);

/* Status word of the last mk_run: 0 ok, 1 grid barrier gave up, 2 a pipeline wait gave up,
 * 3 unsupported extent; and how many grid barriers the run passed. No counterpart in the reference,
 * whose barriers are unbounded. */
void cck_last_status(unsigned int* status, unsigned int* where, unsigned int* barriers);

#ifdef __cplusplus
}
#endif
#endif
