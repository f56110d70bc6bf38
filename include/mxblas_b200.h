/* C ABI of libmxblas_b200.so: FP8 micro-scaled GEMM with fused output group-quantisation for
 * NVIDIA B200 (sm_100a).
 *
 * The entry points stand where the reference has its per-kernel JIT shim
 *     extern "C" void launch(void* a, void* b, void* c, void* as, void* bs, void* cs,
 *                            void* stream, int& __return_code)
 * (mxblas/jit/template.py:114-139, called from mxblas/jit/runtime.py:28-53 with the argument
 * order of mxblas/gemm/kernel_pool.py:113-130). The reference bakes M, N, K, the scale
 * granularity and the layouts into each compiled kernel; here they travel in mxb_problem_t, so one
 * prebuilt library serves every problem. All pointers are raw device pointers unless a function
 * says otherwise, `stream` is a cudaStream_t, every function returns an mxb_status_t and never
 * throws, exits or traps.
 */
#ifndef MXBLAS_B200_H_
#define MXBLAS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXB_ABI_VERSION 1

typedef enum mxb_status {
  MXB_OK = 0,
  MXB_ERR_INVALID = 1,      /* malformed problem (shape, divisibility, alignment, null pointer) */
  MXB_ERR_UNSUPPORTED = 2,  /* well-formed, but no kernel covers it */
  MXB_ERR_WORKSPACE = 3,    /* workspace missing or too small (see mxb_query_workspace) */
  MXB_ERR_CUDA = 4,         /* a CUDA runtime / driver call failed; see mxb_last_cuda_error */
  MXB_ERR_DEVICE = 5        /* a kernel recorded a device-side status (timeout, bad scales) */
} mxb_status_t;

/* element types (mxblas/gemm/descriptor.py:6-11) */
typedef enum mxb_dtype {
  MXB_FP32 = 0,
  MXB_BF16 = 1,
  MXB_FP16 = 2,
  MXB_E4M3 = 3,
  MXB_E5M2 = 4
} mxb_dtype_t;

/* flags */
#define MXB_OUT_QUANT 0x1u            /* output_quant=True (mxblas/jit_kernels/mx_gemm.py:344) */
#define MXB_OUT_TRANSPOSE 0x2u        /* out_transpose=True: C^T [N, M] is written */
#define MXB_OUT_SCALE_TRANSPOSE 0x4u  /* out_scale_transpose=True: C_scale^T [N/QN, M] is written */
#define MXB_OUT_SCALE_POW2 0x8u       /* output scales rounded up to a power of two (extension) */
#define MXB_IN_SCALES_POW2 0x10u      /* caller asserts that all input scales are powers of two */
#define MXB_IN_SCALES_PROBE 0x20u     /* test for power-of-two input scales on the device and use
                                         the native block-scaled MMA when they all are */
#define MXB_LEFT_COL_MAJOR 0x40u      /* left [M, K] is stored column-major: physically [K, M], row pitch lda */
#define MXB_RIGHT_ROW_MAJOR 0x80u     /* right [K, N] is stored row-major: physically [K, N], row pitch ldb */

/* One GEMM problem: the fields of the reference's MXGEMMDescriptor
 * (mxblas/gemm/descriptor.py:84-220) plus the strides that the reference reads from the tensors
 * (mxblas/jit_kernels/mx_gemm.py:160-168).
 *   left        [M, K]  fp8, row-major, row pitch lda (elements); with MXB_LEFT_COL_MAJOR physically [K, M]
 *   right       [K, N]  fp8, column-major view: physically [N, K] with row pitch ldb; with
 *                       MXB_RIGHT_ROW_MAJOR physically [K, N]
 *                       (the reference matches only row-major left x column-major right,
 *                       mxblas/gemm/template.py:70-73; the other three combinations are the operand layouts
 *                       of a backward pass: dX = dY . W with W as stored, dW = dY^T . X)
 *   left_scale  [M/sm, K/sk]  element (i, j) at  i*as_rs + j*as_ks
 *   right_scale [K/sk, N/sn]  element (j, i) at  i*bs_rs + j*bs_ks  (i = column block of N)
 *   out         [M, N] row pitch ldc, or with MXB_OUT_TRANSPOSE [N, M] row pitch ldc
 *   out_scale   [M, N/qn] row pitch ldcs, or with MXB_OUT_SCALE_TRANSPOSE [N/qn, M] row pitch ldcs
 */
typedef struct mxb_problem {
  int32_t m, n, k;
  int32_t sm, sn, sk;    /* rows of left / columns of right / K elements sharing one scale */
  int32_t qm, qn;        /* output quantisation group (qm must be 1); 0, 0 when not quantised */
  int32_t in_dtype;      /* MXB_E4M3 or MXB_E5M2 */
  int32_t out_dtype;     /* MXB_BF16 / MXB_FP16, or MXB_E4M3 / MXB_E5M2 with MXB_OUT_QUANT */
  int32_t scale_dtype;   /* MXB_FP32 / MXB_BF16 / MXB_FP16; also the type of out_scale */
  uint32_t flags;
  int64_t lda, ldb;
  int64_t as_rs, as_ks;
  int64_t bs_rs, bs_ks;
  int64_t ldc, ldcs;
} mxb_problem_t;

/* Kernel configuration; zero / negative fields mean "choose for me". Stands where the reference
 * has its tuning keys (mxblas/jit_kernels/mx_gemm.py:197-291). */
typedef struct mxb_config {
  int32_t bn;         /* MMA N tile: 32, 64, 128, 224 (MX only) or 256 */
  int32_t swap;       /* -1 auto, 0 left on the 128-row MMA axis, 1 right on the 128-row MMA axis */
  int32_t epi_warps;  /* 4 or 8 epilogue warps */
  int32_t raster;     /* tile rows per raster group */
  int32_t splits;     /* split-K factor */
  int32_t ctas;       /* persistent CTAs (0 = one per SM) */
  int32_t cta_pair;   /* 0 auto, 1 one CTA per 128-row tile, 2 CTA pairs on 256 x 256 tiles */
} mxb_config_t;

int mxb_abi_version(void);
const char* mxb_status_string(int status);
/* text of the last CUDA error seen by this thread's calls ("" if none) */
const char* mxb_last_cuda_error(void);

/* Bytes of device scratch the problem needs with this configuration (cfg may be NULL). Scratch
 * holds the re-packed UE8M0 scale factors of the block-scaled MMA path and split-K partial sums.
 * Protocol: the buffer is 256-byte aligned and ZERO-FILLED by the caller before its first use; its
 * first 64 KiB hold counters that every call leaves at zero again, so one buffer can serve any
 * sequence of calls on one stream (calls that overlap on the device need separate buffers). */
int mxb_query_workspace(const mxb_problem_t* problem, const mxb_config_t* cfg, size_t* bytes);

/* Fill `cfg` with the configuration mxb_gemm would choose for `problem`. */
int mxb_default_config(const mxb_problem_t* problem, mxb_config_t* cfg);

/* Enqueue out, out_scale = mx_gemm(left, right, left_scale, right_scale) on `stream`.
 * Replaces launch(a, b, c, as, bs, cs, stream, rc) of mxblas/jit/template.py:114-139.
 * Asynchronous; inputs and workspace must stay valid until the stream reaches the end of the call. */
int mxb_gemm(const mxb_problem_t* problem, const void* left, const void* right, void* out,
             const void* left_scale, const void* right_scale, void* out_scale, void* workspace,
             size_t workspace_bytes, void* stream);

/* Same with an explicit configuration (autotuner, tests). */
int mxb_gemm_cfg(const mxb_problem_t* problem, const mxb_config_t* cfg, const void* left,
                 const void* right, void* out, const void* left_scale, const void* right_scale,
                 void* out_scale, void* workspace, size_t workspace_bytes, void* stream);

/* Grouped GEMM, the expert layers of a mixture-of-experts model: `groups` weight matrices of one shape,
 * right = [groups][N, K] stacked densely (group stride N * ldb) with right_scale = [groups][N/sn, K/sk] stacked the
 * same way; the rows of left [M, K] are sorted by group and padded so that every block of `block_rows` (128 or
 * 256) rows belongs to one group. group_of_block (device memory, M / block_rows ints) names the group of each block;
 * a negative entry skips the block (its rows of out are left untouched). Row r of out is
 * left[r] x right[group of r's block]; scaling, output quantisation and flags as for mxb_gemm, except that
 * MXB_OUT_TRANSPOSE and a row-major right are not supported. block_rows = 256 lets large problems run on CTA
 * pairs. The reference is a single dense GEMM (mxblas/jit_kernels/mx_gemm.py:340-425) and has no counterpart.
 * problem->m is the total number of rows, problem->n the columns of ONE group's weight. */
int mxb_grouped_gemm(const mxb_problem_t* problem, const mxb_config_t* cfg, int groups, const int* group_of_block,
                     int block_rows, const void* left, const void* right, void* out, const void* left_scale,
                     const void* right_scale, void* out_scale, void* workspace, size_t workspace_bytes, void* stream);
int mxb_grouped_query_workspace(const mxb_problem_t* problem, const mxb_config_t* cfg, int groups, int block_rows,
                                size_t* bytes);

/* Host-memory variant: every tensor pointer is HOST memory (pinned memory makes the copies
 * asynchronous). Copies the operands to device staging buffers owned by the library, runs the
 * GEMM in row blocks so that copies and compute overlap, copies the results back and waits.
 * This is the whole-call path a host-resident caller of the reference would time. */
int mxb_gemm_host(const mxb_problem_t* problem, const void* left, const void* right, void* out,
                  const void* left_scale, const void* right_scale, void* out_scale);

/* Scratch built into the library for mxb_gemm_static_scratch, in bytes (held by every GPU that
 * loads the library until the process exits). */
#define MXB_STATIC_SCRATCH_BYTES (8u << 20)

/* mxb_gemm for callers that cannot allocate device memory (a host application with a fixed,
 * pre-planned memory budget, or code that runs where the CUDA allocator must not be entered).
 * Has no counterpart in the reference, whose kernels need no scratch. Same arguments as mxb_gemm
 * without the workspace: split-K partial sums, their counters and re-packed scale factors go to
 * one MXB_STATIC_SCRATCH_BYTES array inside the library. Allocates nothing.
 *   - returns MXB_ERR_WORKSPACE, launching nothing, if the problem needs more scratch than that;
 *   - all calls share the array: calls that overlap on the GPU race and must be serialised;
 *   - the first call on a device performs a one-time address lookup and should be made before any
 *     stream capture is begun on that device. */
int mxb_gemm_static_scratch(const mxb_problem_t* problem, const void* left, const void* right, void* out,
                            const void* left_scale, const void* right_scale, void* out_scale,
                            void* stream);

/* Device-side block quantiser, the step in front of the GEMM: x [m, k] (MXB_FP32 / MXB_BF16 /
 * MXB_FP16, row pitch ldx elements) -> e4m3 codes [m, k] (row pitch ldq bytes) and fp32 scales
 * [m/bm, k/bn] (dense, row-major). Same arithmetic as the reference's host helper block_quant
 * (mxblas/utils.py:66-93): scale = amax / 448 evaluated in x's dtype, 1 for an all-zero block; codes =
 * e4m3(clamp(x / scale, +-448)). Asynchronous on `stream`. */
int mxb_block_quant(const void* x, int x_dtype, long long m, long long k, long long ldx, int bm, int bn,
                    void* codes, long long ldq, float* scales, void* stream);

/* Copy a block of `rows` x `row_bytes` (a multiple of 16; pointers and pitches 16-byte aligned) from `src` into
 * the same position of `copies` (0..7) other buffers, which may be other GPUs' memory mapped into this process
 * (peer access or symmetric memory): plain stores over NVLink, 512 contiguous bytes per warp. An N-sharded run
 * uses it after the GEMM to put a rank's column block of the result into every rank's full result, in place of
 * an all-gather and its re-layout copy; the caller synchronises the ranks before anyone reads. Asynchronous on
 * `stream`. No counterpart in the reference (single GPU). */
int mxb_push_block(const void* src, long long src_pitch, void* const* dsts, int copies, long long dst_pitch,
                   long long rows, long long row_bytes, void* stream);

/* mxb_push_block with a bound on the copy kernel's grid (blocks of 256 threads; 0 = no bound): a caller that
 * runs the push beside a GEMM which leaves a few SMs free sizes it to those SMs (8 blocks each), so that no
 * block of the push waits for, and then delays, the SMs of the GEMM. */
int mxb_push_block_ex(const void* src, long long src_pitch, void* const* dsts, int copies, long long dst_pitch,
                      long long rows, long long row_bytes, int max_blocks, void* stream);

/* mxb_push_block on the copy engines (one 2-D device-to-device copy per destination): uses no SM, so it can
 * run beside a GEMM that occupies all of them. Same arguments; no alignment rule. No counterpart in the
 * reference (single GPU). */
int mxb_push_block_dma(const void* src, long long src_pitch, void* const* dsts, int copies, long long dst_pitch,
                       long long rows, long long row_bytes, void* stream);

/* Read (and optionally clear) the device status word of the current device. Synchronises the
 * device. 0 = no kernel reported a problem; otherwise the first recorded code:
 *   0x100 / 0x200 / 0x300 / 0x400  a bounded wait of the TMA producer / of the MMA warp for operands / of the
 *                                  MMA warp for a drained accumulator / of an epilogue warp gave up
 *   0x500  a split-K or cross-warp quantisation exchange gave up waiting for its peers
 *   0x600  MXB_IN_SCALES_POW2 was asserted but a scale is not a positive power of two
 *   0x700  the self-test below ran its course
 *   0x800  a scale-factor warp of the block-scaled CTA-pair kernel gave up waiting for a TMEM slot
 * A kernel that records a time-out stops issuing work, waits for its copies in flight, frees its
 * tensor memory and returns; its output is then undefined. */
int mxb_device_status(int clear, unsigned int* code);

/* Self-test of the bounded device-side waits (the reference's mbarrier waits spin forever,
 * mxblas/include/mxblas/ptx_wrapper.cuh:50-62): enqueues a one-warp kernel whose wait nothing can
 * satisfy; after about a second the wait gives up, the kernel returns and the status word reads
 * 0x700. The context stays usable. */
int mxb_selftest_wait_timeout(void* stream);

/* Number of GEMM kernels this process has launched through the library (all devices). */
unsigned long long mxb_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* MXBLAS_B200_H_ */
