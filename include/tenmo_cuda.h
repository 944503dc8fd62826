/*
 * libtenmo_cuda.so -- C ABI of the B200 (sm_100a) implementation of tenmo's dense fp32 training path.
 *
 * This is the boundary tenmo's Mojo host binds with OwnedDLHandle / get_function, the same way
 * tenmo/blashandle.mojo:108-251 binds cblas_sgemm.  Each entry point names the reference interface
 * it replaces (paths relative to the reference root).
 *
 * Conventions
 *   - Every data pointer is a DEVICE pointer owned by the caller (tenmo's DeviceBuffer,
 *     device.mojo:325-328).  Outputs are pre-allocated by the caller.  The library owns only its
 *     context, an internal workspace and (optionally) an NCCL communicator.
 *   - Shapes, strides and offsets are in ELEMENTS (int64), row-major, like NDBuffer
 *     (ndbuffer.mojo:66-74).  Data is fp32; class labels are int64 (mnemonics.mojo:63) or int32.
 *   - Calls are asynchronous on the context's stream (tenmo_cuda_set_stream) unless stated.
 *   - Return value: TENMO_OK (0) or a negative tenmo_status; tenmo_cuda_last_error gives the message.
 *     Bad shapes / strides / alignment are rejected on the host before any launch.  Nothing aborts.
 *   - There is no CPU fallback: a layout the tensor-core kernel cannot take runs on the SIMT GPU kernel.
 *   - One host thread per context, and one stream at a time: a context owns ONE workspace, one status / ticket block
 *     and one set of stream-K fix-up flags, so calls that use them (the GEMMs, the column sums, cross-entropy) must
 *     not be in flight on two streams of the same context at once.  Rebinding the context to another stream between
 *     calls is fine when the streams are ordered by events (a side stream that only runs the gradient exchange and
 *     the optimiser, as the trainers do); the library waits for the eight most recently bound streams before it
 *     frees and regrows the workspace and before it reads the status word.  A call that must grow the workspace while
 *     its stream is being captured into a CUDA graph returns TENMO_ERR_STATE: run it once outside the capture first.
 */
#ifndef TENMO_CUDA_H
#define TENMO_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tenmo_ctx tenmo_ctx;

typedef enum {
    TENMO_OK = 0,
    TENMO_ERR_INVALID = -1,      /* bad argument: shape, stride, null pointer, enum out of range */
    TENMO_ERR_CUDA = -2,         /* a CUDA runtime/driver call failed; message has the CUDA error string */
    TENMO_ERR_UNSUPPORTED = -3,  /* valid request this build cannot serve (e.g. algo forced on a bad layout) */
    TENMO_ERR_NOMEM = -4,        /* workspace allocation failed */
    TENMO_ERR_NCCL = -5,         /* NCCL load / call failed */
    TENMO_ERR_TIMEOUT = -6,      /* a bounded device-side wait gave up; see tenmo_cuda_check_device_status */
    TENMO_ERR_STATE = -7         /* call made in the wrong state (e.g. dp call before tenmo_dp_init) */
} tenmo_status;

/* ---- context ------------------------------------------------------------------------------------
 * Replaces tenmo's GPU/DeviceContext wrapper (device.mojo:87-90) for the purposes of this path. */
int tenmo_cuda_init(int device, tenmo_ctx** out);
void tenmo_cuda_destroy(tenmo_ctx* ctx);
const char* tenmo_cuda_last_error(tenmo_ctx* ctx); /* ctx may be NULL: the calling thread's last error from a call without a context */
const char* tenmo_cuda_version(void);
/* Stream handle of the caller's DeviceContext (a cudaStream_t, taken verbatim: NULL is CUDA's default
 * stream).  A new context runs on a stream of its own; TENMO_STREAM_OWN selects that one again. */
#define TENMO_STREAM_OWN ((void*)(intptr_t)-1)
int tenmo_cuda_set_stream(tenmo_ctx* ctx, void* cuda_stream);
/* The persistent tensor-core GEMM launches one CTA per SM.  While a collective runs beside it on another
 * stream (data-parallel gradient exchange) its CTAs need SMs of their own: leave `n` SMs out of the GEMM
 * grid (0 restores the full grid).  No counterpart in the reference (single stream, no collectives). */
int tenmo_cuda_reserve_sms(tenmo_ctx* ctx, int n);
/* DeviceContext.synchronize (the `sync=True` argument of every launcher, matmul_kernel.mojo:277). */
int tenmo_cuda_synchronize(tenmo_ctx* ctx);
int tenmo_cuda_device_info(tenmo_ctx* ctx, int* sm_count, int* cc_major, int* cc_minor, int* sm_clock_khz);
/* Synchronises, then reads the device status word kernels set when a bounded wait (mbarrier) gave up.
 * Returns TENMO_OK or TENMO_ERR_TIMEOUT; the word is cleared. */
int tenmo_cuda_check_device_status(tenmo_ctx* ctx);
/* Launches a one-thread kernel that waits, with the bounded wait of the GEMM kernels and a limit of limit_us
 * microseconds (1 .. 1 000 000), on a barrier nothing ever arrives on.  The kernel gives up, raises the status word and
 * returns like any other; the next tenmo_cuda_check_device_status then answers TENMO_ERR_TIMEOUT and the context stays
 * usable.  No reference counterpart: it exists so that the expiry path of the device-side waits can be exercised
 * without a fault. */
int tenmo_cuda_wait_probe(tenmo_ctx* ctx, int limit_us);
/* Counts kernel launches made through this context since the last reset (bookkeeping for benchmarks). */
int64_t tenmo_cuda_launch_count(tenmo_ctx* ctx, int reset);
/* Device timing of the GEMM main kernels (not the split / reduction helpers around them): between
 * begin and end every such launch is bracketed by a CUDA event pair on the context's stream (at most
 * 4096 launches are recorded).  end synchronises and returns the number of launches and the sum of
 * their durations.  Takes the place of the reference's hand timing with perf_counter_ns
 * (profile_gpu.mojo:36-65). */
int tenmo_cuda_profile_begin(tenmo_ctx* ctx);
int tenmo_cuda_profile_end(tenmo_ctx* ctx, int64_t* launches, double* total_ms);

/* ---- GEMM ---------------------------------------------------------------------------------------
 * A strided, possibly batched matrix operand: element (b..., i, j) lives at
 *   ptr[offset + sum_d coord_d * batch_stride[d] + i*row_stride + j*col_stride].
 * Batch dims are right-aligned and broadcast NumPy-style; an operand's batch stride is applied only
 * where its own batch dim is > 1 (matmul_cpu.mojo:706-724). */
#define TENMO_MAX_BATCH_RANK 6 /* max_rank 8 (mnemonics.mojo:45) minus the two matrix dims */
typedef struct {
    const float* ptr;
    int64_t offset;
    int64_t row_stride, col_stride;
    int32_t batch_rank;
    int64_t batch_shape[TENMO_MAX_BATCH_RANK];
    int64_t batch_stride[TENMO_MAX_BATCH_RANK];
} tenmo_mat;

enum { TENMO_ALGO_AUTO = -1, TENMO_ALGO_SIMT_FP32 = 0, TENMO_ALGO_TC_3XTF32 = 1 };
enum { TENMO_ACT_NONE = 0, TENMO_ACT_RELU = 1, TENMO_ACT_SIGMOID = 2 };

/* C[b] = act( A[b] . B[b] + bias ) (+ C[b] when beta == 1);  A is (M,K), B is (K,N), C is the
 * contiguous (total_batch, M, N) output.
 * Replaces NDBuffer.matmul_2d / matmul_nd GPU branch (ndbuffer.mojo:2404-2501) and
 * MatmulNdGpu.launch (kernels/matmul_kernel.mojo:128-283); with transposed stride views as operands it
 * is also the two backward GEMMs of Matmul2dBackward / MatmulNdBackward (matmul.mojo:24-54,101-137).
 *   algo   TENMO_ALGO_SIMT_FP32: strict fp32, every output one k-ascending fmaf chain (bit-identical to
 *          matmul_cpu.mojo paths 1a/1b).  TENMO_ALGO_TC_3XTF32: tcgen05 tensor cores, three TF32 products
 *          per fp32 product.  TENMO_ALGO_AUTO picks the tensor-core kernel when the layout allows
 *          (unit inner stride on one axis of each operand, 16-byte aligned rows) and the problem is
 *          large enough, else SIMT.
 *   beta   0 or 1.  beta == 1 is the Gradbox accumulate `grad += incoming` (ancestry.mojo:83-84,
 *          kernels/binary_inplace_ops_kernel.mojo) folded into the epilogue.
 *   bias   N floats or NULL: the Linear bias add (net.mojo:194-203, binary_ops_kernel.mojo:408-458).
 *   act    applied after the bias: ReLU (relu.mojo:97-141) or Sigmoid (buffers.mojo:1147-1152).
 *   aux    optional, same shape as C: the fp32 0/1 ReLU mask (x > 0) that relu.mojo stores for backward.
 *   colsum optional, N floats, 2-D only: colsum[n] (+)= sum_k B[k,n], i.e. the bias gradient when this
 *          call is dW = X^T . dY (broadcast.mojo:66-88); follows beta. */
int tenmo_gemm_f32(tenmo_ctx* ctx, int algo, int64_t M, int64_t N, int64_t K, const tenmo_mat* A,
                   const tenmo_mat* B, float* C, float beta, const float* bias, int act, float* aux,
                   float* colsum);
/* The same GEMM with every option in one struct (zero-initialise it; NULL opts = all defaults), plus what a
 * host that chains GEMMs can use to stop paying for the 3xTF32 operand split more than once per tensor:
 *   a_lo, b_lo  lo planes of the operands' STORAGE as written by tenmo_split_lo_f32 or by an earlier call's
 *               c_lo (a transposed view shares its storage's plane); NULL = split inside the call.
 *               Ignored by the SIMT kernel.
 *   c_lo        optional output: lo plane of the stored result, row-major, leading dimension N rounded up
 *               to a multiple of 4, batches back to back -- ready to be the a_lo / b_lo of the next GEMM.
 *   mul_mask    optional (total_batch, M, N) multiplier applied to act(A.B + bias) before beta / store: with
 *               the ReLU mask of the layer below, dX = (dY . W^T) * mask is ReLUBackward (relu.mojo:19-46)
 *               fused into Matmul2dBackward's dA GEMM (matmul.mojo:33-41).
 * No counterpart in the reference, which runs each of these as a separate kernel. */
typedef struct {
    float beta;
    const float* bias;
    int act;
    float* aux;
    float* colsum;
    const float* a_lo;
    const float* b_lo;
    float* c_lo;
    const float* mul_mask;
    const float* bias_m; /* optional M floats added per ROW: the per-channel bias when a convolution runs as
                            W(C_out, C_in*KH*KW) . patches^T.  The SIMT kernel starts its accumulators at it,
                            as the reference's convolution does (cnn.mojo:435). */
} tenmo_gemm_opts;
int tenmo_gemm_f32_ex(tenmo_ctx* ctx, int algo, int64_t M, int64_t N, int64_t K, const tenmo_mat* A,
                      const tenmo_mat* B, float* C, const tenmo_gemm_opts* opts);
/* lo plane (x minus x truncated to TF32, rounded to TF32) of a (rows, cols) view X with one unit-stride axis,
 * 16-byte aligned rows and batch dims that collapse to one stride.  Written in the order of X's storage:
 * `outer` lines of `inner` floats, lines padded to a multiple of 4, batches back to back; `capacity` is the
 * size of lo_out in floats and must cover that. */
int tenmo_split_lo_f32(tenmo_ctx* ctx, const tenmo_mat* X, int64_t rows, int64_t cols, float* lo_out, int64_t capacity);
/* Which kernel the last tenmo_gemm_f32 call on this context ran: TENMO_ALGO_SIMT_FP32 or _TC_3XTF32. */
int tenmo_gemm_last_algo(tenmo_ctx* ctx);
/* Name of the kernel that call launched: "gemm_tc_kernel", "gemm_simt_tma_kernel" (strict fp32, TMA-staged tiles),
 * "gemm_simt_kernel" (strict fp32, register-staged: any strides) or "gemm_skinny_kernel" (strict fp32, a result of at
 * most 32 columns over a contraction of 512 or more); "" before the first call.  No reference
 * counterpart; tests and benchmarks use it to state which path was measured. */
const char* tenmo_gemm_last_kernel(tenmo_ctx* ctx);
/* Pieces of the stream-K tail of that launch: when the tiles of a tensor-core GEMM do not fill the last wave of CTAs,
 * the k-range of the last tiles is cut into this many equal pieces (one per CTA) and the partial accumulators are
 * added in ascending k by the piece that holds a tile's end; 0 = every tile was computed whole (always 0 for the
 * strict-fp32 kernels, whose results must not depend on the machine).  TENMO_TC_STREAMK=0 in the environment turns
 * it off.  No reference counterpart. */
int tenmo_gemm_last_stream_k(tenmo_ctx* ctx);
/* 1 when that launch ran as CTA pairs: two CTAs on neighbouring SMs share a 256 x 256 tile (tcgen05.mma.cta_group::2,
 * each staging half of the right-hand tile; three shared-memory stages instead of two).  Chosen when the product has at
 * least two such tiles per pair of SMs; TENMO_TC_PAIR=0 / 1 in the environment forces it off / on.  No reference
 * counterpart. */
int tenmo_gemm_last_pair(tenmo_ctx* ctx);

/* ---- matrix @ vector, vector @ matrix ---------------------------------------------------------------
 * y[i] = sum_k A[i,k] x[k] (+ y[i] when beta == 1): MatrixVectorMulNd.forward (matrixvector.mojo:205-285), and
 * y[j] = sum_k x[k] A[k,j]: VectorMatmulNd.forward (vectormatrix.mojo:210-340); with g in place of x they are also the
 * vector gradients of the two backward passes (matrixvector.mojo:15-201, vectormatrix.mojo:14-206).  A is one
 * (M,K) / (K,N) matrix view (batch_rank 0; a batched caller loops, as the reference's forward does) with a unit
 * stride on at least one axis; x has element stride incx >= 1; y is contiguous.  HBM-bound kernels that read A once;
 * sums are not in the reference's k-ascending order, so results agree with it to rounding (the bit-identical form is
 * tenmo_gemm_f32 with a unit dimension and the strict-fp32 algorithm, which also serves a matrix without a
 * unit-stride axis: these two return TENMO_ERR_UNSUPPORTED for it). */
int tenmo_gemv_f32(tenmo_ctx* ctx, int64_t M, int64_t K, const tenmo_mat* A, const float* x, int64_t incx, float* y,
                   float beta);
int tenmo_vecmat_f32(tenmo_ctx* ctx, int64_t K, int64_t N, const float* x, int64_t incx, const tenmo_mat* A, float* y,
                     float beta);

/* ---- elementwise neighbours of the GEMM (un-fused forms, for a host that calls op by op) ---------- */
/* out[m,n] = x[m,n] + bias[n]; Adder.forward bias case (addition.mojo:71-112,
 * binary_ops_kernel.mojo:778-807).  out may alias x. */
int tenmo_add_bias_f32(tenmo_ctx* ctx, const float* x, const float* bias, float* out, int64_t M, int64_t N);
/* out[i] += in[i]; Gradbox accumulate (gradbox.mojo:1358-1364, ndbuffer.mojo:1714-1719). */
int tenmo_add_inplace_f32(tenmo_ctx* ctx, float* out, const float* in, int64_t n);
/* x[i] = value; NDBuffer.fill used by zero_grad (optim.mojo:546-581, device.mojo:215-227). */
int tenmo_fill_f32(tenmo_ctx* ctx, float* x, float value, int64_t n);
/* ReLU.forward: out = max(x,0), mask = x>0 ? 1 : 0 (relu.mojo:50-95, unary_ops_kernel.mojo:220-298).
 * mask may be NULL. */
int tenmo_relu_fwd_f32(tenmo_ctx* ctx, const float* x, float* out, float* mask, int64_t n);
/* ReLUBackward: dx = g * mask, (+= when beta == 1) (relu.mojo:19-46). */
int tenmo_relu_bwd_f32(tenmo_ctx* ctx, const float* g, const float* mask, float* dx, float beta, int64_t n);
/* Sigmoid.forward y = 1/(1+exp(-x)) (sigmoid.mojo:32-53, unary_ops_kernel.mojo:146-218). */
int tenmo_sigmoid_fwd_f32(tenmo_ctx* ctx, const float* x, float* y, int64_t n);
/* SigmoidBackward dx = g*y*(1-y) (sigmoid.mojo:9-29, binary_ops_kernel.mojo:29-68). */
int tenmo_sigmoid_bwd_f32(tenmo_ctx* ctx, const float* g, const float* y, float* dx, float beta, int64_t n);

/* ---- reductions ---------------------------------------------------------------------------------
 * out[n] = sum_m x[m*ldx + n] (+ out[n] when beta == 1).  The bias gradient
 * (broadcast.mojo:66-88 -> sum_mean_reduction.mojo:37-158, kernels/reduction_kernel.mojo:136-214) and,
 * with M = leading batch and N = the rest, sum_over_broadcasted_axes (sum_mean_reduction.mojo:184-211). */
int tenmo_colsum_f32(tenmo_ctx* ctx, const float* x, int64_t M, int64_t N, int64_t ldx, float* out, float beta);

/* The same column sum for callers that must not let the library allocate (no counterpart in the
 * reference).  A host that owns all device memory through its own pool, or a loop that cannot afford
 * the device-wide synchronisation of cudaMalloc / cudaFree, cannot use the entry point above, which
 * grows a workspace on first use.  This one needs no context and calls no allocator: its scratch (the
 * partial sums and ticket counters of the split kernel) is a fixed array inside the loaded module,
 * about 4 MiB, held by every GPU that loads the library until the process exits.
 *   - Limit: N <= 16384 columns (any M, any ldx >= N); beyond that it returns TENMO_ERR_UNSUPPORTED and
 *     tenmo_cuda_last_error(NULL) says so.
 *   - Runs on the CURRENT device, on `cuda_stream` (a cudaStream_t; NULL = default stream).
 *   - The first call on each device is the set-up call: it resolves the array's device address
 *     (cudaGetSymbolAddress), which under CUDA's lazy module loading is also the moment the module is loaded
 *     and the array comes into existence on that device, so that one call may synchronise the device.  Make it
 *     during start-up, outside any stream capture; every later call allocates and synchronises nothing.  The
 *     set-up is safe to race from several host threads.
 *   - All calls share the one array.  What must start at zero is cleared on the stream before each
 *     launch, but two calls whose kernels overlap on the GPU (different streams) race on it. */
int tenmo_colsum_f32_static(const float* x, int64_t M, int64_t N, int64_t ldx, float* out, float beta,
                            void* cuda_stream);

/* ---- convolution as GEMM and max pooling, NCHW ---------------------------------------------------------
 * The reference's Conv2d (cnn.mojo:290-950) pads the image (pad.mojo) and then convolves directly; here the
 * padding is an argument (pad = 0 reproduces the pre-padded contract) and the arithmetic is a GEMM between
 * the kernel tensor viewed as (C_out, C_in*KH*KW) and the patch matrix these helpers produce / consume.
 *   im2col   patches[(n,oy,ox), (c,ky,kx)] = x[n, c, oy*stride - pad + ky*dilation, ox*stride - pad + kx*dilation],
 *            zero outside the image; patches is (N*Ho*Wo, C*KH*KW) row-major (the patch extraction of
 *            compute_kernel_gradient, cnn.mojo:716-778).
 *   col2im   adjoint of im2col: dx (N,C,H,W) (+)= gather of dpatches (compute_input_gradient, cnn.mojo:812-950).
 *   channel_sum   out[c] (+)= sum over n and the S trailing elements of g viewed as (N, C, S)
 *            (compute_bias_gradient, cnn.mojo:664-714).
 *   maxpool2d fwd  k x k window, first maximum wins (strict >), argmax = y*W + x inside the (n,c) plane or -1
 *            (pooling.mojo:301-402); bwd  dx = 0 then dx[argmax] += g (pooling.mojo:25-107). */
int tenmo_conv_out_size(int64_t in, int k, int stride, int dilation, int pad, int64_t* out);
/* The convolution as an implicit GEMM: the patch matrix is never written, the image region a tile of outputs reads is
 * staged in shared memory and the multiplies gather from there (3x3 / stride 1 / dilation 1 kernels; other geometries
 * run plain gather kernels).  Strict fp32.
 *   fwd         out[n,co,oy,ox] = act(bias[co] + sum over (ci,ky,kx) ascending of x * weight): Conv2dFused.forward
 *               (cnn.mojo:404-507), the accumulator starting at the bias (cnn.mojo:435) -- bit-identical to that chain.
 *               act: TENMO_ACT_NONE or TENMO_ACT_RELU; mask (optional, shape of out) receives the 0/1 ReLU mask
 *               (relu.mojo:97-141).  bias may be NULL.
 *   bwd_input   dx (+)= the input gradient (compute_input_gradient, cnn.mojo:812-950), gathered instead of scattered.
 *   bwd_weight  dW (+)= grad . patches and db (+)= per-channel sum of grad (compute_kernel_gradient / compute_bias_gradient,
 *               cnn.mojo:716-809, 664-714); per-slab partial sums are added in slab order, so results repeat run to run.
 *   g_mask (optional, shape of g): the 0/1 ReLU mask of the layer's output; the kernels use g * g_mask, which fuses
 *               ReLUBackward (relu.mojo:19-46) into the load.  beta: 0 or 1 (accumulate into the outputs). */
int tenmo_conv2d_fwd_f32(tenmo_ctx* ctx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const float* weight,
                         const float* bias, int64_t Cout, int KH, int KW, int stride, int dilation, int pad, int act,
                         float* out, float* mask);
int tenmo_conv2d_bwd_input_f32(tenmo_ctx* ctx, const float* g, const float* g_mask, const float* weight, int64_t N, int64_t C,
                               int64_t H, int64_t W, int64_t Cout, int KH, int KW, int stride, int dilation, int pad,
                               float* dx, float beta);
int tenmo_conv2d_bwd_weight_f32(tenmo_ctx* ctx, const float* x, const float* g, const float* g_mask, int64_t N, int64_t C,
                                int64_t H, int64_t W, int64_t Cout, int KH, int KW, int stride, int dilation, int pad,
                                float* dW, float* db, float beta);
int tenmo_im2col_f32(tenmo_ctx* ctx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW,
                     int stride, int dilation, int pad, float* patches);
int tenmo_col2im_f32(tenmo_ctx* ctx, const float* dpatches, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW,
                     int stride, int dilation, int pad, float* dx, float beta);
int tenmo_channel_sum_f32(tenmo_ctx* ctx, const float* g, int64_t N, int64_t C, int64_t S, float* out, float beta);
int tenmo_maxpool2d_fwd_f32(tenmo_ctx* ctx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int k, int stride,
                            int pad, float* out, int64_t* argmax);
int tenmo_maxpool2d_bwd_f32(tenmo_ctx* ctx, const float* g, const int64_t* argmax, int64_t N, int64_t C, int64_t H,
                            int64_t W, int64_t Ho, int64_t Wo, float* dx);

/* ---- softmax over the last axis (the step between the two GEMMs of an attention block) --------------
 * Forward y = exp(x - max) / sum (SoftmaxNdBuffer.softmax, softmax.mojo:30-48); x has leading dimension ldx,
 * y is contiguous (M, C).  Backward dx = y * (g - sum_c(g * y)) (+= when beta == 1)
 * (SoftmaxBackwardDelegate, softmax.mojo:206-213). */
int tenmo_softmax_fwd_f32(tenmo_ctx* ctx, const float* x, int64_t ldx, float* y, int64_t M, int64_t C);
int tenmo_softmax_bwd_f32(tenmo_ctx* ctx, const float* y, const float* g, float* dx, float beta, int64_t M, int64_t C);

/* ---- softmax cross-entropy, class-index targets ---------------------------------------------------
 * reduction: 0 mean, 1 sum, 2 none (shared/__init__.mojo:4-40).
 * Forward (crossentropy.mojo:285-432, kernels/crossentropy_fused_kernel.mojo:39-160): per row max,
 * exp, sum, loss; softmax_out (M,C) is kept for backward (may be NULL).  loss_dev receives 1 float
 * (mean/sum) or M floats (none); valid_count_dev 1 int32 (rows whose label != ignore_index).
 * Labels outside [0,C) other than ignore_index are a caller error (the host validates them,
 * crossentropy.mojo:114-134); such a row contributes nothing and sets the device status word. */
int tenmo_ce_fwd_f32(tenmo_ctx* ctx, const float* logits, int64_t ld_logits, const void* labels,
                     int label_is_i64, int64_t M, int64_t C, int64_t ignore_index, float label_smoothing,
                     int reduction, float* softmax_out, float* loss_dev, int32_t* valid_count_dev);
/* Backward (crossentropy.mojo:664-823, crossentropy_fused_kernel.mojo:192-275):
 * dlogits = (softmax - (1-ls)*onehot - ls/C) * valid * upstream / (mean ? valid_count : 1)
 * (+= when beta == 1).  upstream_dev: 1 float (mean/sum) or M floats (none); NULL means 1.0. */
int tenmo_ce_bwd_f32(tenmo_ctx* ctx, const float* softmax, const void* labels, int label_is_i64, int64_t M,
                     int64_t C, int64_t ignore_index, float label_smoothing, int reduction,
                     const float* upstream_dev, const int32_t* valid_count_dev, float* dlogits, float beta);
/* Forward and backward in one call, for a loss that is the root of the backward pass (loss.backward() right after
 * criterion(pred, labels): crossentropy.mojo:1360-1391 then 664-823).  Same arguments and the same bits as
 * tenmo_ce_fwd_f32 followed by tenmo_ce_bwd_f32 with beta = 0; softmax_out is required.  A small batch
 * (M <= 256 and M*C <= 16384, the MNIST- and CIFAR-shaped configurations) is ONE launch: the CTA that finishes the
 * loss and the valid count also writes dlogits.  Larger batches run the two kernels. */
int tenmo_ce_fwd_bwd_f32(tenmo_ctx* ctx, const float* logits, int64_t ld_logits, const void* labels,
                         int label_is_i64, int64_t M, int64_t C, int64_t ignore_index, float label_smoothing,
                         int reduction, float* softmax_out, float* loss_dev, int32_t* valid_count_dev,
                         const float* upstream_dev, float* dlogits);

/* ---- optimiser ----------------------------------------------------------------------------------
 * SGD.step dense path for n_tensors parameters in ONE launch (optim.mojo:405-543,
 * kernels/sgd_kernel.mojo:7-128):  g' = g*grad_scale; if wd>0: g' += p*wd;
 * momentum>0: v = momentum*v + g'; p -= lr*v;   momentum==0: p -= lr*g'.
 * p, g, v are HOST arrays of n_tensors device pointers (v may be NULL when momentum == 0). */
int tenmo_sgd_step_f32(tenmo_ctx* ctx, int n_tensors, float* const* p, const float* const* g, float* const* v,
                       const int64_t* numel, float lr, float momentum, float weight_decay, float grad_scale);
/* The same step that also leaves the 3xTF32 lo plane of the updated parameters: p_lo[t] (may be NULL per tensor)
 * receives tf32_lo of the first lo_numel[t] updated elements of tensor t, in the same order (the layout of
 * tenmo_split_lo_f32 for a matrix whose rows are a multiple of 4 long).  Saves the separate split pass over the
 * weights after every update; the parameters come out bit-identical to tenmo_sgd_step_f32. */
int tenmo_sgd_step_lo_f32(tenmo_ctx* ctx, int n_tensors, float* const* p, const float* const* g, float* const* v,
                          const int64_t* numel, float* const* p_lo, const int64_t* lo_numel, float lr, float momentum,
                          float weight_decay, float grad_scale);

/* ---- accuracy -----------------------------------------------------------------------------------
 * Accuracy.compute (accuracy.mojo:7-85, kernels/accuracy_kernel.mojo:9-84): rows whose first-index
 * argmax (strict >) equals the label.  Works for any M.  correct_dev: 1 int64 on the device, overwritten.
 * If correct_host != NULL the call synchronises and copies the count there. */
int tenmo_accuracy_f32(tenmo_ctx* ctx, const float* logits, int64_t ld_logits, const void* labels,
                       int label_is_i64, int64_t M, int64_t C, int64_t* correct_dev, int64_t* correct_host);

/* ---- data parallel (no counterpart in the reference: README.md:472-473 lists it as future work) ----
 * One process per GPU.  Rank 0 obtains an id with tenmo_dp_get_unique_id and shares it out of band;
 * every rank then calls tenmo_dp_init.  tenmo_dp_allreduce_sum_f32 sums `count` floats in place over
 * all ranks on the context's stream (NCCL over NVLink / NVSwitch). */
#define TENMO_DP_ID_BYTES 128
int tenmo_dp_get_unique_id(tenmo_ctx* ctx, void* id_out, size_t id_bytes);
int tenmo_dp_init(tenmo_ctx* ctx, int rank, int world, const void* id, size_t id_bytes);
int tenmo_dp_allreduce_sum_f32(tenmo_ctx* ctx, float* buf, int64_t count);
int tenmo_dp_finalize(tenmo_ctx* ctx);

/* The same exchange as one kernel of this library over NVLink peer memory (no NCCL; no reference counterpart).
 * Every rank allocates the gradient bucket inside the library (tenmo_dp_p2p_alloc: `count` floats, zeroed; the
 * pointer is the caller's to fill, the memory stays the library's) and receives TENMO_DP_P2P_HANDLE_BYTES of CUDA IPC
 * handles; the ranks share their handle blocks out of band, rank-major, and every rank calls tenmo_dp_p2p_connect
 * with all of them.  tenmo_dp_p2p_allreduce_sum_f32 then sums bucket[offset, offset + count) over the ranks in place,
 * asynchronously on the context stream: every element is added once, in rank order, by the rank that owns its
 * shard, so all ranks end with identical bits.  All ranks must make the same calls in the same order.  Its waits on the
 * peers are bounded (2 s) and report through
 * tenmo_cuda_check_device_status.  At most 8 ranks, all on one node.  tenmo_dp_p2p_close unmaps and frees; the ranks
 * must have finished using each other's buckets (a host barrier) before any of them calls it. */
#define TENMO_DP_P2P_HANDLE_BYTES 128
int tenmo_dp_p2p_alloc(tenmo_ctx* ctx, int64_t count, float** buf_out, void* handles_out, size_t handles_bytes);
int tenmo_dp_p2p_connect(tenmo_ctx* ctx, int rank, int world, const void* all_handles, size_t handles_bytes);
int tenmo_dp_p2p_allreduce_sum_f32(tenmo_ctx* ctx, int64_t offset, int64_t count);
/* The exchange and SGD.step (optim.mojo:405-543) as one kernel with the optimiser sharded over the ranks.  The bucket
 * holds the gradients of the range at [grad_offset, +count) and the parameters at [param_offset, +count) (disjoint
 * ranges of the same allocation, so that the peers can read both).  Per call: every rank adds the W gradient copies of
 * its shard in rank order, applies g' = g*grad_scale (+ p*wd); v = momentum*v + g'; p -= lr*v to its shard of the
 * parameters -- the arithmetic of tenmo_sgd_step_f32, bit for bit -- and then copies the other ranks' updated shards,
 * so every rank ends with identical parameters.  v: this rank's velocities for the range (count floats, device
 * memory of the caller; only the own shard is read and written, so a rank holds the momentum of 1/W of the
 * parameters).  p_lo / lo_count: optional 3xTF32 lo plane of the first lo_count updated parameters of the range,
 * written as the parameters land (see tenmo_sgd_step_lo_f32).  The gradient range is left as it was.  Same rules as
 * the all-reduce: same calls in the same order on every rank, one call in flight per context, bounded waits.
 * Both kernels keep their call counter on the device, so a captured CUDA graph that contains them can be replayed. */
int tenmo_dp_p2p_sgd_step_f32(tenmo_ctx* ctx, int64_t grad_offset, int64_t param_offset, int64_t count, float* v,
                              float* p_lo, int64_t lo_count, float lr, float momentum, float weight_decay,
                              float grad_scale);
/* Form of the exchange kernels.  Off (default): 128 CTAs x 512 threads, for an exchange that runs with nothing beside it
 * (fastest by itself).  On: 128 CTAs x 128 threads at no more than 85 registers, small enough to share an SM with the
 * persistent GEMM CTA, for a host that overlaps the exchange with the backward GEMMs.  Every rank must choose the same. */
int tenmo_dp_p2p_set_coresident(tenmo_ctx* ctx, int on);
int tenmo_dp_p2p_close(tenmo_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* TENMO_CUDA_H */
