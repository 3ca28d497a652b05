/*
 * qste_b200 -- C ABI of the B200 (sm_100a) binary-layer kernels.
 *
 * One shared library, libqste_b200.so.  Every entry point takes raw DEVICE
 * pointers, explicit sizes and a CUDA stream; it enqueues work on that stream and
 * returns without synchronising.  The caller owns every buffer, including the
 * scratch ("workspace") whose size the matching *_workspace() function reports.
 * The library allocates no device memory.
 *
 * Return value: 0 on success, a negative qste_status otherwise
 * (qste_b200_status_string() names it).  Nothing here falls back to a CPU path.
 *
 * Bit layout shared by every packed operand: least-significant bit first; byte b
 * of a row holds columns 8b..8b+7; a set bit means "value >= 0", i.e. weight +1;
 * the row pitch is ceil(columns / 8) bytes; pad bits are written as 0.
 *
 * Each declaration cites the interface of the reference (BleedingXiko/QSTE,
 * paths relative to that project) that it stands in for.
 */
#ifndef QSTE_B200_H
#define QSTE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QSTE_B200_ABI_VERSION 1

/* cudaStream_t without pulling in the CUDA headers */
typedef struct CUstream_st* qste_stream_t;

typedef enum {
  QSTE_OK = 0,
  QSTE_ERR_SHAPE = -1,      /* a size is negative, zero where it may not be, or inconsistent */
  QSTE_ERR_DTYPE = -2,      /* unknown qste_dtype */
  QSTE_ERR_ALIGNMENT = -3,  /* a pointer is not aligned as documented */
  QSTE_ERR_WORKSPACE = -4,  /* workspace missing or smaller than *_workspace() reports */
  QSTE_ERR_CUDA = -5,       /* a CUDA runtime/driver call failed (launch, tensor map, attribute) */
  QSTE_ERR_UNSUPPORTED = -6,/* argument combination this build does not implement */
  QSTE_ERR_NULL = -7,       /* a required pointer is NULL */
  QSTE_ERR_ARCH = -8,       /* the current device is not compute capability 10.x */
  QSTE_ERR_LIMIT = -9       /* size beyond a documented fixed maximum */
} qste_status;

typedef enum {
  QSTE_F32 = 0,
  QSTE_F16 = 1,
  QSTE_BF16 = 2
} qste_dtype;

/* Which GEMM implementation a projection call should use. */
typedef enum {
  QSTE_PATH_AUTO = 0,   /* tcgen05 tensor-core kernel when the shape allows it, else the others */
  QSTE_PATH_SIMT = 1,   /* generic CUDA-core kernel (any shape) */
  QSTE_PATH_TENSOR = 2, /* tcgen05/TMEM kernel; QSTE_ERR_UNSUPPORTED when the shape does not fit */
  QSTE_PATH_STREAM = 3  /* the small-batch kernels only (QSTE_ERR_UNSUPPORTED where none applies): forward by look-up
                           tables for 1-2 tokens (1-4 of fp32) or weights expanded in registers for 3-32 tokens of
                           a 16-bit type; qste_b200_linear_backward_evidence in one launch for 1-128 samples */
} qste_path;

int qste_b200_abi_version(void);
const char* qste_b200_status_string(int status);
/* Text of the last CUDA error this library saw on the calling thread ("" if none). */
const char* qste_b200_last_cuda_error(void);
/* Number of kernels this library has launched in this process so far. */
unsigned long long qste_b200_launch_count(void);
/* Which kernel family the calling thread's last qste_b200_packed_linear_affine ran: "lut" (1-2
 * tokens), "mma" (3-32 tokens, 16-bit), "stream", "tensor" (tcgen05), "simt", or "" before the
 * first call.  A diagnostic for tests and benchmarks; the reference has no counterpart. */
const char* qste_b200_last_forward_kernel(void);
/* The tensor-core GEMMs are persistent kernels with one block per SM.  A collective that runs
 * beside them on another stream (the evidence all-reduce of data-parallel training) finds no
 * free SM until a GEMM ends.  This sets how many SMs the GEMMs launched FROM THE CALLING THREAD
 * leave free from now on (0 = none, the default; the environment variable
 * QSTE_B200_RESERVED_SMS gives a thread's initial value) and returns the previous setting.
 * It changes the GEMMs' grid and so the size *_workspace() reports: set it before the
 * workspace query of the call it is meant for.  No counterpart in the reference, whose GEMMs
 * are cuBLAS calls. */
int qste_b200_set_reserved_sms(int count);

/* ---- workspaces --------------------------------------------------------------
 * A workspace is caller-owned device memory, 256-byte aligned, at least as large as the
 * matching *_workspace() reports, and used by one call at a time (one workspace per stream).
 * Its first 256 bytes are a header that the library reads and updates across calls; the caller
 * must ZERO THE HEADER ONCE, before the first call that uses the buffer (cudaMemset of 256
 * bytes), and carry it over if it replaces the buffer by a larger one.  Layout (all uint64):
 *   bytes   0..7    number of bounded device-side waits that gave up (0 in a healthy run; a
 *                   GEMM whose wait gave up returns QSTE_OK all the same, and its output is
 *                   incomplete: check this counter wherever the stream is synchronised anyway)
 *   bytes   8..15   flip count of the last coordinate_update
 *   bytes  64..191  per-role cycle counters of the GEMM (filled when QSTE_B200_TC_PROFILE is set)
 *   bytes 192..199  the GEMM's work-item counter, zero between launches: a non-zero start makes a
 *                   launch skip tiles, which is why the header must start zeroed
 *   bytes 200..207  where the first wait gave up: source line << 32 | block << 16 | thread
 * The rest is scratch with no meaning between calls.
 *
 * Process-wide state the library keeps (everything else lives in caller memory): per-device
 * caches of the SM count, the compute capability, "shared-memory attribute set" flags and the
 * resident-cluster capacity of the pair kernel (written once each, identical values from any
 * thread); the driver entry point of cuTensorMapEncodeTiled; a launch counter; per-thread: the
 * last CUDA error text and the reserved-SM setting.  The environment switches QSTE_B200_TC_*
 * (test and profiling only) are read once, at the first GEMM of the process. */

/* ---- packing --------------------------------------------------------------- */

/* bits of (coordinate >= 0).  Reference: kernels.pack_coordinate,
 * src/qste/kernels/loader.py:285-289, cpu.cpp:207-238. */
int qste_b200_pack_coordinate(const int8_t* coordinate, int64_t rows, int64_t columns,
                              uint8_t* packed, qste_stream_t stream);

/* Per row: offset = mean(x); bits of (x - offset >= 0); scale = mean|x - offset|,
 * with the reference's fp32 summation order, so the bits match its CPU kernel.
 * values is [rows, columns] of `dtype`, row-major, contiguous.
 * Reference: kernels.pack_affine_rows, loader.py:278-282, cpu.cpp:143-203. */
int qste_b200_pack_affine_rows(const void* values, int dtype, int64_t rows, int64_t columns,
                               uint8_t* packed, float* offset, float* scale,
                               qste_stream_t stream);

/* One bit per element of a bool (1 byte per element) matrix.
 * Reference: kernels.pack_bits, loader.py:256-260, cpu.cpp:246-277. */
int qste_b200_pack_bits(const uint8_t* mask, int64_t rows, int64_t columns, uint8_t* packed,
                        qste_stream_t stream);

/* out = values where the bit is set, 0 elsewhere; values/out are `dtype`.
 * Reference: kernels.apply_bits, loader.py:263-267, cpu.cpp:281-316. */
int qste_b200_apply_bits(const void* values, int dtype, const uint8_t* packed, int64_t rows,
                         int64_t columns, void* out, qste_stream_t stream);

/* Dense view of packed bits in `dtype`: +-1 when zero_one == 0 (kernels.unpack_rows,
 * loader.py:247-253, cpu.cpp:318-325), 0/1 otherwise (kernels.unpack_bits,
 * loader.py:270-275). */
int qste_b200_unpack_rows(const uint8_t* packed, int64_t rows, int64_t columns, void* out,
                          int dtype, int zero_one, qste_stream_t stream);

/* ---- projections ----------------------------------------------------------- */

/* Y[m, r] = (sum_c X[m, c] * sign[r, c]) * scale[r] + bias[r]   (bias may be NULL)
 * X is [samples, columns] of `dtype`; Y is [samples, rows] of `out_dtype`.
 * Reference: kernels.packed_linear_affine, loader.py:292-296, cpu.cpp:342-371. */
size_t qste_b200_packed_linear_affine_workspace(int64_t samples, int64_t rows, int64_t columns,
                                                int dtype, int path);
int qste_b200_packed_linear_affine(const void* inputs, int dtype, int64_t samples,
                                   const uint8_t* packed, const float* scale, const float* bias,
                                   int64_t rows, int64_t columns, void* out, int out_dtype,
                                   int path, void* workspace, size_t workspace_bytes,
                                   qste_stream_t stream);

/* dX[m, c] = sum_r (dY[m, r] * row_scale[r]) * sign[r, c]   (row_scale may be NULL)
 * Reference: kernels.packed_transpose, loader.py:299-303, cpu.cpp:375-410. */
size_t qste_b200_packed_transpose_workspace(int64_t samples, int64_t rows, int64_t columns,
                                            int dtype, int path);
int qste_b200_packed_transpose(const void* inputs, int dtype, int64_t samples,
                               const uint8_t* packed, const float* row_scale, int64_t rows,
                               int64_t columns, void* out, int out_dtype, int path,
                               void* workspace, size_t workspace_bytes, qste_stream_t stream);

/* E[r, c] = sum_m (dY[m, r] * sample_scale[m]) * sign(x)[m, c], always fp32.
 * `packed` holds the activation bits, [samples, ceil(columns/8)]; sample_scale may be NULL.
 * Reference: kernels.evidence_from_packed, loader.py:306-312, cpu.cpp:416-456. */
size_t qste_b200_evidence_from_packed_workspace(int64_t samples, int64_t rows, int64_t columns,
                                                int dtype, int path);
int qste_b200_evidence_from_packed(const void* grad, int dtype, int64_t samples, int64_t rows,
                                   const uint8_t* packed, const float* sample_scale,
                                   int64_t columns, float* evidence, int path, void* workspace,
                                   size_t workspace_bytes, qste_stream_t stream);

/* The whole evidence side of a converted Linear's backward in one call
 * (src/qste/functional.py:186-193 with decoded_evidence at :118-145):
 *   E0[r, c]   = sum_m dY[m, r] * (act_scale[m] * sign(x)[m, c] + act_offset[m])
 *   g_scale[r] = sum_c E0[r, c] * sign(W)[r, c]
 *   evidence   = E0 * weight_scale[r]                       (fp32 [rows, columns])
 *   g_bias[r]  = sum_m dY[m, r]                              (skipped when g_bias is NULL)
 * aux is the saved [2, samples] fp32 tensor: offsets then scales.
 * Batches of 1-128 samples (columns a multiple of 128) run as ONE kernel: look-up tables on the CUDA
 * cores up to 16 samples (fp32 throughout), warp-level MMAs with one fp16 rounding per term above;
 * larger batches on the tensor-core tiles. */
size_t qste_b200_linear_backward_evidence_workspace(int64_t samples, int64_t rows,
                                                    int64_t columns, int dtype, int path);
int qste_b200_linear_backward_evidence(const void* grad, int dtype, int64_t samples, int64_t rows,
                                       const uint8_t* act_bits, const float* aux, int64_t columns,
                                       const uint8_t* weight_bits, const float* weight_scale,
                                       float* evidence, float* g_scale, float* g_bias, int path,
                                       void* workspace, size_t workspace_bytes,
                                       qste_stream_t stream);

/* Everything backward of a converted Linear computes, in one call: dX (as
 * qste_b200_packed_transpose) and evidence / g_scale / g_bias (as
 * qste_b200_linear_backward_evidence).  Doing both at once lets one pass over dY produce the
 * bias gradient, the offset correction and dY's largest magnitude, and lets both GEMMs share one
 * fp16 re-encoding of a bf16 dY.  grad_input is [samples, columns] of `grad_input_dtype`.
 * Reference: QSTELinearFn.backward, src/qste/functional.py:173-194. */
size_t qste_b200_linear_backward_workspace(int64_t samples, int64_t rows, int64_t columns, int dtype);
int qste_b200_linear_backward(const void* grad, int dtype, int64_t samples, int64_t rows,
                              const uint8_t* weight_bits, const float* weight_scale, int64_t columns,
                              const uint8_t* act_bits, const float* aux, void* grad_input,
                              int grad_input_dtype, float* evidence, float* g_scale, float* g_bias,
                              void* workspace, size_t workspace_bytes, qste_stream_t stream);

/* qste_b200_linear_backward for a caller that overlaps the backward with work on another
 * stream.  The evidence product runs first; when `evidence_ready` (a cudaEvent_t the caller
 * created, or NULL) is given it is recorded on `stream` as soon as evidence, g_scale and g_bias
 * are complete, before the dX product is enqueued, so an all-reduce or a coordinate update on a
 * second stream can wait for that event and run beside dX.  grad_input may be NULL: dX is then
 * not computed at all (a layer whose input needs no gradient).
 * Reference: QSTELinearFn.backward, src/qste/functional.py:173-194 together with the reducer
 * call of QSTEOptimizer._apply, src/qste/optim.py:156-178, which it lets start early. */
int qste_b200_linear_backward_staged(const void* grad, int dtype, int64_t samples, int64_t rows,
                                     const uint8_t* weight_bits, const float* weight_scale,
                                     int64_t columns, const uint8_t* act_bits, const float* aux,
                                     void* grad_input, int grad_input_dtype, float* evidence,
                                     float* g_scale, float* g_bias, void* evidence_ready,
                                     void* workspace, size_t workspace_bytes, qste_stream_t stream);

/* out[r] = sum_c matrix[r, c] * sign[r, c], fp32.
 * Reference: kernels.packed_row_inner, loader.py:315-319, cpu.cpp:460-496. */
int qste_b200_packed_row_inner(const float* matrix, const uint8_t* packed, int64_t rows,
                               int64_t columns, float* out, qste_stream_t stream);

/* out[i, :] = sign[ids[i], :] * scale[ids[i]] in `out_dtype`.  Ids outside [0, rows) set
 * *bad_id (a device int32, pre-zeroed by the caller) to 1 and write zeros.
 * Reference: kernels.packed_embedding, loader.py:322-326, cpu.cpp:499-538. */
int qste_b200_packed_embedding(const int64_t* ids, int64_t count, const uint8_t* packed,
                               const float* scale, int64_t rows, int64_t columns, void* out,
                               int out_dtype, int32_t* bad_id, qste_stream_t stream);

/* ---- packed activations ----------------------------------------------------- */

/* Smooth activation with an int8 derivative tape, forward: for every row of `inputs`
 * ([rows, columns] of `dtype`, row-major, contiguous)
 *   outputs    = f(inputs)                                     (same dtype)
 *   scale[r]   = max(max_c |f'(inputs[r, c])|, 1e-8) / 127     (fp32)
 *   derivative = clamp(rint(f'(inputs) / scale[r]), -127, 127) (int8 [rows, columns])
 * in one pass over the row.  `kind` is a qste_activation; `parameter` is alpha (ELU, CELU) or
 * beta (Softplus) and ignored otherwise.  columns * 4 bytes must fit in shared memory
 * (QSTE_ERR_LIMIT beyond 51200 columns).
 * Reference: _SmoothFn.forward, src/qste/nn.py:483-502, with the derivatives of :392-470. */
typedef enum {
  QSTE_ACT_GELU = 0, QSTE_ACT_GELU_TANH = 1, QSTE_ACT_SILU = 2, QSTE_ACT_TANH = 3,
  QSTE_ACT_SIGMOID = 4, QSTE_ACT_ELU = 5, QSTE_ACT_CELU = 6, QSTE_ACT_SELU = 7,
  QSTE_ACT_SOFTPLUS = 8, QSTE_ACT_MISH = 9, QSTE_ACT_HARDSWISH = 10
} qste_activation;
int qste_b200_smooth_forward(const void* inputs, int dtype, int64_t rows, int64_t columns, int kind,
                             double parameter, void* outputs, int8_t* derivative, float* scale,
                             qste_stream_t stream);

/* ... and backward: grad_inputs = grad * (derivative * scale[r]), each product rounded to
 * `dtype` as the reference's torch expression rounds it.
 * Reference: _SmoothFn.backward, src/qste/nn.py:504-507. */
int qste_b200_smooth_backward(const void* grad, int dtype, const int8_t* derivative,
                              const float* scale, int64_t rows, int64_t columns, void* grad_inputs,
                              qste_stream_t stream);

/* ---- coordinate optimizer --------------------------------------------------- */

/* One optimizer step for one surface, in place on coordinate / packed / moment_q /
 * moment_scale / row_v / col_v; `gradient` (fp32 [rows, columns]) is consumed as
 * scratch.  moment_scale, row_v, col_v are IEEE fp16.  The arithmetic follows the
 * reference's CPU kernel operation by operation (including the order of every fp32
 * sum), so the int8 outputs and the packed bits are the reference's.
 *   step_device    : optional device int64 read at run time instead of `step`
 *   update_enabled : optional device uint8; 0 turns the call into a no-op
 *   flips_out      : optional device int64 that receives the number of flipped signs
 * The flip count is also left in the workspace at byte offset 8 (int64).
 * Reference: kernels.coordinate_update, loader.py:329-368, cpu.cpp:578-808,
 * cuda.py:1705-1812 (device-side step / flips / update_enabled). */
size_t qste_b200_coordinate_update_workspace(int64_t rows, int64_t columns, int64_t block_size);
int qste_b200_coordinate_update(float* gradient, int8_t* coordinate, uint8_t* packed,
                                int8_t* moment_q, uint16_t* moment_scale, uint16_t* row_v,
                                uint16_t* col_v, int64_t rows, int64_t columns, double beta1,
                                double beta2, double update_clip, double coordinate_lr,
                                int64_t block_size, int64_t seed, int64_t step,
                                const int64_t* step_device, const uint8_t* update_enabled,
                                int64_t* flips_out, void* workspace, size_t workspace_bytes,
                                qste_stream_t stream);

/* The same optimizer step for callers that cannot hand the library any scratch memory:
 * a host that binds this C ABI from a runtime whose device memory is one pre-planned arena
 * it does not own, or code that runs where entering the CUDA allocator is off limits (a
 * locked memory budget, a driver callback).  The scratch lives inside the library image as
 * a fixed device array (about 3 MB per GPU, held from library load to process exit), so
 * the call allocates nothing and takes no workspace.  Inputs, outputs and the in-place
 * state are still the caller's, exactly as in qste_b200_coordinate_update.
 *   - Limits: rows <= 16384, columns <= 16384 and ceil(rows * columns / block_size) <=
 *     262144; anything larger returns QSTE_ERR_LIMIT and touches nothing.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture.
 *   - Every call on a device shares the one array.  Calls are safe back to back on one
 *     stream; two calls that may run at the same time on the GPU (different streams) race.
 *   - flips_out is required here if the flip count is wanted: there is no workspace to
 *     read it back from.
 * No counterpart in the reference: its kernels allocate through torch. */
int qste_b200_coordinate_update_static(float* gradient, int8_t* coordinate, uint8_t* packed,
                                       int8_t* moment_q, uint16_t* moment_scale, uint16_t* row_v,
                                       uint16_t* col_v, int64_t rows, int64_t columns, double beta1,
                                       double beta2, double update_clip, double coordinate_lr,
                                       int64_t block_size, int64_t seed, int64_t step,
                                       const int64_t* step_device, const uint8_t* update_enabled,
                                       int64_t* flips_out, qste_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* QSTE_B200_H */
