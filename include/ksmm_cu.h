/*
 * ksmm_cu.h -- C ABI of the B200-native Kronecker-sparse matrix multiplication
 * (KSMM) library, libksmm_cu.so.
 *
 * The reference project has no C ABI.  Each entry point below names the
 * reference interface it stands in for (paths relative to the reference
 * checkout).  All pointers are plain device pointers unless the name says
 * "host"; no torch type appears anywhere in this file.
 *
 * Conventions shared by every call
 *   - one factor has a pattern (a, b, c, d); weights ("values") are in the
 *     reference's kernel format: a row-major (a*d*c, b) matrix whose element
 *     [((i_a*d + i_d)*c + k), j] is W[i_a, j, k, i_d]
 *     (src/ksmm_py/layer/kronecker_sparse/interface.py:65-69,
 *      src/ksmm_cu/src/template_sparse_mm.cu:362-394);
 *   - batch-last (bs_last = 1): input is (a*c*d, batch) row-major, output is
 *     (a*b*d, batch); batch-first (bs_last = 0): input is (batch, a*c*d),
 *     output is (batch, a*b*d);
 *   - inputs are borrowed, outputs are caller-owned and fully overwritten;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); every call is asynchronous with respect to the host and
 *     ordered on that stream, except the *_host calls, which return after the
 *     result is in host memory;
 *   - the return value is a ksmm_status_t; on failure ksmm_cu_last_error()
 *     gives a message for the calling thread.  The library never aborts the
 *     process (the reference asserts: kernel_bs_first_float.cuh:18,
 *     kernel.cu:123-125).
 */
#ifndef KSMM_CU_H_
#define KSMM_CU_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define KSMM_API __attribute__((visibility("default")))
#else
#define KSMM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  KSMM_OK = 0,
  KSMM_ERR_BAD_ARGUMENT = 1,   /* null pointer, non-positive size, bad enum   */
  KSMM_ERR_UNSUPPORTED = 2,    /* dtype / layout combination not implemented  */
  KSMM_ERR_CUDA = 3,           /* a CUDA runtime or driver call failed        */
  KSMM_ERR_WORKSPACE = 4,      /* workspace missing or too small              */
  KSMM_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait gave up          */
  KSMM_ERR_NO_DEVICE = 6       /* no sm_100 device is visible                 */
} ksmm_status_t;

/* Element types.  The strings the reference passes through pybind
 * ("torch.float32", "torch.float16", "torch.float8_e4m3fn"; kernel.cu:66,83,103)
 * map onto these in the Python layer. */
typedef enum {
  KSMM_F32 = 0,
  KSMM_F16 = 1,
  KSMM_BF16 = 2,
  KSMM_F8E4M3 = 3
} ksmm_dtype_t;

/* Kernel families (for ksmm_forward_desc_t.algo and the tuner). */
typedef enum {
  KSMM_ALGO_AUTO = 0,   /* cached tuner choice, else heuristic                */
  KSMM_ALGO_SIMT = 1,   /* FFMA register-tiled kernel, any shape/alignment     */
  KSMM_ALGO_TC = 2,     /* tcgen05 + TMEM + TMA kernels (fp32, 16-bit, fp8)    */
  KSMM_ALGO_CONVERT = 3 /* batch-first, d > 1: transpose, batch-last kernel, transpose */
} ksmm_algo_t;

/* Full description of one factor multiplication. */
/* Element-wise function fused into the epilogue (the reference has none: its
 * callers apply activations as separate PyTorch kernels). */
typedef enum {
  KSMM_ACT_NONE = 0,
  KSMM_ACT_GELU = 1,   /* 0.5 x (1 + erf(x / sqrt 2)), torch.nn.functional.gelu's default */
  KSMM_ACT_RELU = 2
} ksmm_activation_t;

typedef struct {
  const void* input;
  const void* values;     /* kernel-format weights, (a*d*c, b) row-major       */
  void* output;
  const void* bias;       /* optional, a*b*d elements of out_dtype, or NULL    */
  int64_t batch;
  int32_t a, b, c, d;
  int32_t in_dtype;       /* ksmm_dtype_t of input and values                  */
  int32_t out_dtype;      /* ksmm_dtype_t of output (F8 not allowed)           */
  int32_t bs_last;        /* 1 = batch-last, 0 = batch-first                   */
  int32_t algo;           /* ksmm_algo_t                                       */
  int32_t config;         /* tile configuration index inside the family, -1 = auto */
  float alpha;            /* output = act(alpha * (K x) + bias); fp8: s_x * s_w */
  int32_t activation;     /* ksmm_activation_t applied last in the epilogue    */
  void* scratch;          /* optional device memory for the paths that need a  */
  size_t scratch_bytes;   /* second copy of a tensor (ksmm_cu_layout_scratch_bytes); */
                          /* NULL = a library-owned buffer per (device, stream) */
  const void* residual;   /* optional tensor shaped, laid out and typed like   */
                          /* the output, added last: out = act(...) + residual */
} ksmm_forward_desc_t;

/* Library version: major*10000 + minor*100 + patch. */
KSMM_API int ksmm_cu_version(void);

/* Message for the last failure on the calling thread ("" if none). */
KSMM_API const char* ksmm_cu_last_error(void);
KSMM_API const char* ksmm_cu_status_string(int status);

/*
 * One factor, output dtype = input dtype, alpha = 1, no bias.
 * Replaces the C++-linkage launchers
 *   void best_kernel_bs_{first,last}_{float,half}(T* input, T* values, T* output,
 *        int batch_size, int a, int b, int c, int d, dim3&, dim3&)
 * (src/ksmm_py/layer/kronecker_sparse/kernel_bs_first_float.cuh:8-21,
 *  kernel_bs_last_half.cuh:8-21) and the dtype/layout switch around them
 * (kernel.cu:40-127).  Argument order follows those launchers: input, values,
 * output, batch, a, b, c, d.
 */
KSMM_API int ksmm_cu_forward(const void* input, const void* values, void* output,
                    int64_t batch, int a, int b, int c, int d,
                    int dtype, int bs_last, void* stream);

/*
 * One factor with every option (mixed output type, scale, bias, forced kernel
 * family / tile configuration).  Same reference counterpart as
 * ksmm_cu_forward; the fp8 path is what the reference's empty branch
 * (kernel.cu:66-82) and its standalone fp8 kernels
 * (src/ksmm_cu/src/template_kernels_fp8.cuh:22-370) were meant to provide,
 * with per-tensor scales folded into alpha and fp32 accumulation.
 */
KSMM_API int ksmm_cu_forward_ex(const ksmm_forward_desc_t* desc, void* stream);

/*
 * Device memory (bytes) that ksmm_cu_forward_ex needs beside input, weights
 * and output for this problem under the current dispatch: non-zero only for
 * batch-first factors with d > 1 that run through a layout conversion or a
 * regrouping pass (the reference's kernels index such inputs directly with
 * strided scalar accesses, template_kernels_half.cuh:402-413, and need none).
 * A caller that passes that much in desc->scratch keeps the call free of any
 * allocation; with scratch == NULL the library uses its own buffer for the
 * (device, stream) pair, grown on demand and released by
 * ksmm_cu_release_scratch (which synchronises the device first).
 */
KSMM_API size_t ksmm_cu_layout_scratch_bytes(const ksmm_forward_desc_t* desc);
KSMM_API int ksmm_cu_release_scratch(void);

/*
 * A chain of factors: patterns[4*f .. 4*f+3] = (a,b,c,d) of factor f, applied
 * f = 0 first, as KSLinear.forward_bs_{first,last} loops over its factors
 * (interface.py:193-211, 269-291) and post_process adds the bias once
 * (interface.py:451-467).  `workspace` holds the intermediate activations;
 * its size comes from ksmm_cu_chain_workspace_bytes (0 for a single factor).
 */
KSMM_API size_t ksmm_cu_chain_workspace_bytes(int nfactors, const int32_t* patterns,
                                     int64_t batch, int dtype);
/* Intermediates plus the layout scratch of the factors that need one in the
 * given layout: with a workspace of this size a chain call never allocates.
 * (With the smaller size above, such factors use the library-owned buffer of
 * the calling stream.) */
KSMM_API size_t ksmm_cu_chain_workspace_bytes_ex(int nfactors, const int32_t* patterns,
                                        int64_t batch, int dtype, int bs_last);
KSMM_API int ksmm_cu_chain_forward(const void* input, const void* const* values, void* output,
                          const void* bias, void* workspace, size_t workspace_bytes,
                          int64_t batch, int nfactors, const int32_t* patterns,
                          int dtype, int bs_last, void* stream);
/* Same call with an element-wise activation (ksmm_activation_t) applied after the bias in the
 * last factor's epilogue; no reference counterpart (the reference's callers run the activation
 * as a separate PyTorch kernel). */
KSMM_API int ksmm_cu_chain_forward_act(const void* input, const void* const* values, void* output,
                              const void* bias, void* workspace, size_t workspace_bytes,
                              int64_t batch, int nfactors, const int32_t* patterns,
                              int dtype, int bs_last, int activation, void* stream);

/*
 * A chain whose output layout may differ from its input layout, e.g. the two
 * KSLinear layers of an MLP with the activations between them kept batch-last
 * while the network around them is batch-first (the reference fixes one
 * layout per layer, interface.py:134, 193-345, and pays for interleaved blocks
 * in every batch-first factor with d > 1).  The library plans a layout for
 * every intermediate: 16-bit and fp32 factors with d = 1 read one layout and
 * write the other inside the kernel, at no cost (fp32: b a multiple of 32, c
 * of 4, batch of 32); where no such factor exists the tensor
 * at the chain's end is transposed.  ksmm_cu_chain_forward and
 * ksmm_cu_chain_forward_act are this call with out_bs_last = bs_last, and use
 * the same planner, so their intermediates may be batch-last inside a
 * batch-first chain.  Workspace: ..._workspace_bytes_layouts.
 */
KSMM_API size_t ksmm_cu_chain_workspace_bytes_layouts(int nfactors, const int32_t* patterns,
                                             int64_t batch, int dtype, int bs_last, int out_bs_last);
KSMM_API int ksmm_cu_chain_forward_layouts(const void* input, const void* const* values, void* output,
                                  const void* bias, void* workspace, size_t workspace_bytes,
                                  int64_t batch, int nfactors, const int32_t* patterns,
                                  int dtype, int bs_last, int out_bs_last, int activation,
                                  void* stream);

/*
 * The chain call with every option in one descriptor, among them a residual:
 * out = act(K_n ... K_1 x + bias) + residual, the `x + ff(x)` of a transformer
 * block (src/ksmm_py/model/vit.py:574-577 adds it as a separate PyTorch
 * kernel).  `residual` has the output's shape, layout and type; the 16-bit
 * tensor kernel adds it in its epilogue, other kernels in a pass after them.
 * out_layout: 0 = the input's layout, 1 = batch-first, 2 = batch-last.
 */
typedef struct {
  const void* input;
  const void* const* values;   /* nfactors kernel-format weights                 */
  void* output;
  const void* bias;            /* optional, out features                         */
  const void* residual;        /* optional, shaped like the output               */
  void* workspace;             /* ksmm_cu_chain_workspace_bytes_layouts          */
  size_t workspace_bytes;
  int64_t batch;
  int32_t nfactors;
  const int32_t* patterns;     /* 4 * nfactors integers                          */
  int32_t dtype;               /* ksmm_dtype_t (not fp8)                         */
  int32_t bs_last;             /* layout of the input                            */
  int32_t out_layout;          /* 0 = as the input, 1 = batch-first, 2 = batch-last */
  int32_t activation;          /* ksmm_activation_t                              */
} ksmm_chain_desc_t;
KSMM_API int ksmm_cu_chain_forward_desc(const ksmm_chain_desc_t* desc, void* stream);

/*
 * Several problems of one pattern in one call ("groups"): the q, k and v
 * projections of an attention layer apply the same patterns to the same input
 * (src/ksmm_py/model/get_vit.py:164-215 builds to_q, to_k, to_v from one
 * pattern list; src/ksmm_py/model/vit.py:477-478 calls them one after the
 * other on the same x).  Here the `groups` weight sets are stacked,
 * values = (groups, a*d*c, b), the outputs are stacked, output = (groups,
 * a*b*d, batch) batch-last or (groups, batch, a*b*d) batch-first (each group's
 * result is a contiguous tensor), and the input is either one tensor read by
 * every group (shared_input = 1: the first factor of q/k/v) or stacked like
 * the output (shared_input = 0: the later factors of the three chains).
 * `bias` is NULL or groups * a*b*d elements.  The 16-bit tensor-core kernel
 * runs all groups in one launch, the groups of an input tile side by side so
 * that the tile is fetched from HBM once; other cases run group by group.
 */
KSMM_API int ksmm_cu_grouped_forward(const void* input, const void* values, void* output,
                                     const void* bias, int64_t batch, int a, int b, int c, int d,
                                     int dtype, int bs_last, int groups, int shared_input,
                                     void* stream);
/* The same for chains: every group applies the same `patterns`; values[f] is
 * the stacked (groups, a*d*c, b) weight of factor f; the input is shared by
 * the groups, the output is stacked.  Workspace: groups times
 * ksmm_cu_chain_workspace_bytes_ex of one chain. */
KSMM_API int ksmm_cu_grouped_chain_forward(const void* input, const void* const* values, void* output,
                                           const void* bias, void* workspace, size_t workspace_bytes,
                                           int64_t batch, int nfactors, const int32_t* patterns,
                                           int dtype, int bs_last, int groups, void* stream);

/*
 * Backward of one factor.  The reference has none: Kernel.backward is a stub
 * that calls an undefined kernel.backward
 * (src/ksmm_py/layer/kronecker_sparse/kernel.py:323-329).
 *
 * ksmm_cu_backward_input: grad_input = K^T grad_output, i.e. the same
 *   multiplication with pattern (a, c, b, d) and every b x c block
 *   transposed.  The workspace receives the transposed blocks (a*b*c*d
 *   elements) and, where the (a, c, b, d) multiplication needs one, its layout
 *   scratch; ..._workspace_bytes gives the total (the first part is
 *   mandatory, without the second the library-owned scratch is used).
 *   grad_output has the forward output's shape, grad_input the input's.
 * ksmm_cu_backward_weights: grad_values[(i*d + l)*c + k, j] = sum over the
 *   batch of grad_output[(i, j, l), n] * input[(i, k, l), n], in the kernel
 *   format and type of the weights (fp32 accumulation).  16-bit batch-last
 *   and batch-first d = 1 problems run on the tensor cores with the batch
 *   split over CTAs; they need ..._workspace_bytes of fp32 partial sums
 *   (without it, and for every other case, a plain FFMA kernel runs).
 */
KSMM_API size_t ksmm_cu_backward_input_workspace_bytes(int64_t batch, int a, int b, int c, int d,
                                                       int dtype, int bs_last);
KSMM_API int ksmm_cu_backward_input(const void* grad_output, const void* values, void* grad_input,
                                    void* workspace, size_t workspace_bytes, int64_t batch,
                                    int a, int b, int c, int d, int dtype, int bs_last, void* stream);
KSMM_API size_t ksmm_cu_backward_weights_workspace_bytes(int64_t batch, int a, int b, int c, int d,
                                                         int dtype, int bs_last);
KSMM_API int ksmm_cu_backward_weights(const void* input, const void* grad_output, void* grad_values,
                                      void* workspace, size_t workspace_bytes, int64_t batch,
                                      int a, int b, int c, int d, int dtype, int bs_last, void* stream);

/*
 * ksmm_cu_chain_forward without any allocation: the intermediate activations
 * live in a fixed array of KSMM_CU_STATIC_SCRATCH_BYTES that is part of the
 * library image (each GPU that loads the library carries it until the process
 * exits).  No counterpart in the reference.
 *
 * It is meant for callers that cannot call cudaMalloc or grow a framework
 * allocator at the point of the call: code that runs between other people's
 * kernels on a latency-critical stream, where an allocation would synchronise
 * the device, or an embedding host that gives plugins a fixed memory budget
 * and forbids allocation after start-up.  Inputs, weights and the output are
 * still the caller's buffers.
 *
 *   - the array holds the chain's intermediates and, for batch-first factors
 *     that run through a layout conversion, their transposed input and output
 *     (ksmm_cu_chain_workspace_bytes_ex gives the total).  A chain that needs
 *     more is rejected with KSMM_ERR_WORKSPACE before anything is launched;
 *     the call never falls back to an allocation.  The default size holds one
 *     38.5 MB intermediate, e.g. the two-factor KS-ViT-B MLP layers in fp16 or
 *     the batch-last README layer in fp32 at batch 25088;
 *   - the first call on a device resolves the array's device address, which
 *     makes the driver load the part of the library image that holds the
 *     array (its free-memory reading drops by the array's size then, once);
 *     make that call before starting a stream capture;
 *   - all calls on one GPU share the array, and it keeps the previous call's
 *     contents: calls that may overlap on the GPU (different streams) race and
 *     must be serialised by the caller.  Nothing has to be cleared between
 *     calls, every intermediate is overwritten in full.
 */
#define KSMM_CU_STATIC_SCRATCH_BYTES (40u * 1024u * 1024u)
KSMM_API int ksmm_cu_chain_forward_static(const void* input, const void* const* values,
                                          void* output, const void* bias, int64_t batch,
                                          int nfactors, const int32_t* patterns, int dtype,
                                          int bs_last, void* stream);

/*
 * Host-memory variant of ksmm_cu_chain_forward: input, values and output are
 * HOST buffers; the call stages them through device memory that the library
 * owns (grown on demand, reused across calls), runs the chain and returns
 * after the output has been copied back.  This is the call a C user without
 * its own device buffers makes; it stands in for the standalone driver's
 * cudaMalloc / cudaMemcpy / launch / cudaMemcpy sequence
 * (src/ksmm_cu/src/template_sparse_mm.cu:443-457, 545-784, 800-803).
 * `device` is the CUDA device ordinal.
 */
KSMM_API int ksmm_cu_chain_forward_host(const void* host_input, const void* const* host_values,
                               void* host_output, const void* host_bias,
                               int64_t batch, int nfactors, const int32_t* patterns,
                               int dtype, int bs_last, int device);
/*
 * The same call split in two, so that a caller with several inputs keeps both
 * directions of the host link busy: ..._host_async enqueues the copies and the
 * chain and returns a ticket at once; ksmm_cu_host_wait blocks until that
 * call's output is complete in host memory.  Calls are served in order, and
 * the upload of one call overlaps the download of the one before it (the
 * standalone driver of the reference copies, launches and copies back one
 * input at a time: template_sparse_mm.cu:443-457, 800-803).  The host buffers
 * of a call (input, values, bias, output) must stay valid and untouched until
 * its ticket has been waited for; pinned (page-locked) buffers are what makes
 * the copies asynchronous.  A ticket of 0 (empty batch) needs no wait.
 */
KSMM_API int ksmm_cu_chain_forward_host_async(const void* host_input, const void* const* host_values,
                                     void* host_output, const void* host_bias,
                                     int64_t batch, int nfactors, const int32_t* patterns,
                                     int dtype, int bs_last, int device, uint64_t* ticket);
KSMM_API int ksmm_cu_host_wait(uint64_t ticket);

/*
 * Tile-configuration introspection and tuning.  Replaces the offline
 * exhaustive search of src/ksmm_cu/long_run.sh:178-229 and the generated
 * .best tables (kernel_bs_last_float.best etc.): candidates are compiled in,
 * timed in-process with CUDA events and cached per
 * (dtype, layout, a, b, c, d, batch).
 *
 * ksmm_cu_num_configs: number of tile configurations of a kernel family.
 *   (fp32 in the tensor-core family: 0 = output tile chosen by a cost rule,
 *   1, 2, 3 = output tiles of 128, 96, 64 columns.)
 * ksmm_cu_config_supported: 1 if (algo, config) can run this problem.
 * ksmm_cu_tune: times every supported candidate on the given buffers (which
 *   must be valid for the problem; output is overwritten), stores the winner
 *   in the in-process cache, and reports it.  best_ms may be NULL.  Every
 *   timed launch (nrepeats per candidate, at most 64) starts with a cold L2:
 *   the call allocates a buffer of 1.5x the cache for its own duration and
 *   overwrites it before each launch, outside the timed interval.  An
 *   offline call: it allocates, synchronises the stream and frees.
 * ksmm_cu_set_choice / ksmm_cu_get_choice: write / read the cache directly,
 *   so that a saved table can be re-loaded without re-timing.
 * ksmm_cu_default_choice: what KSMM_ALGO_AUTO runs for this problem (a cached
 *   choice if there is one, else the heuristic): the kernel family, its
 *   configuration (-1 = the family's own default) and whether the call goes
 *   through the layout-conversion path (transpose, batch-last kernel,
 *   transpose).  Pointers in `desc` are only checked for alignment.
 * KSMM_ALGO_CONVERT (one configuration, 0) is that conversion path as a
 *   family of its own, so that the tuner can time it against the direct
 *   kernels and a saved table can name it.  A cached choice is used only when
 *   it can run on the pointers of the actual call; otherwise the heuristic
 *   decides, as if nothing were cached.
 */
KSMM_API int ksmm_cu_num_configs(int algo);
KSMM_API int ksmm_cu_config_supported(int algo, int config, int64_t batch, int a, int b, int c, int d,
                             int in_dtype, int out_dtype, int bs_last);
KSMM_API int ksmm_cu_tune(const ksmm_forward_desc_t* desc, int nrepeats, void* stream,
                 int* best_algo, int* best_config, float* best_ms);
KSMM_API int ksmm_cu_set_choice(int64_t batch, int a, int b, int c, int d, int in_dtype, int out_dtype,
                       int bs_last, int algo, int config);
KSMM_API int ksmm_cu_get_choice(int64_t batch, int a, int b, int c, int d, int in_dtype, int out_dtype,
                       int bs_last, int* algo, int* config);
KSMM_API int ksmm_cu_default_choice(const ksmm_forward_desc_t* desc, int* algo, int* config,
                           int* via_transpose);
/* Removes one cached choice (the heuristic decides again), or the whole cache when batch < 0. */
KSMM_API int ksmm_cu_clear_choice(int64_t batch, int a, int b, int c, int d, int in_dtype, int out_dtype,
                         int bs_last);

/*
 * Synchronises `stream` and returns KSMM_ERR_DEVICE_TIMEOUT if a kernel
 * launched earlier on the current device gave up one of its bounded waits
 * (the flag is then cleared), KSMM_OK otherwise.  The reference has no
 * counterpart: its launchers never check a CUDA or device status
 * (kernel.cu:40-127).
 */
KSMM_API int ksmm_cu_check_device(void* stream);

/* Number of kernel launches issued by this library in the calling process
 * since load (all threads); used by the benchmark to report its launch count. */
KSMM_API uint64_t ksmm_cu_launch_count(void);

/* Number of device allocations (cudaMalloc) the library itself has made in
 * this process: layout scratch, the staging buffers of the *_host calls, the
 * FFMA probe, the cache-flush buffer of ksmm_cu_tune.  A caller that must not allocate at call time can assert that
 * the count does not move across its calls. */
KSMM_API uint64_t ksmm_cu_alloc_count(void);

/*
 * Test hook for the timeout path: launches one warp that waits, through the
 * same bounded wait as the kernels, on a barrier nothing will ever signal, with
 * a limit of `limit_cycles` SM cycles (at most 4e9).  The wait runs out, the
 * warp returns, and the next ksmm_cu_check_device reports
 * KSMM_ERR_DEVICE_TIMEOUT (code 99).  Nothing faults and the context stays
 * usable.  No counterpart in the reference.
 */
KSMM_API int ksmm_cu_debug_wait_probe(int64_t limit_cycles, void* stream);

/* FP32 FFMA throughput probe: runs a register-resident FMA loop on every SM
 * and returns the measured TFLOP/s in *tflops (the fp32 roofline denominator,
 * which no vendor library reports). */
KSMM_API int ksmm_cu_measure_ffma_peak(float* tflops, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KSMM_CU_H_ */
