/*
 * CPU oracle: a C++ restatement of tenmo's own CPU implementation of the dense
 * fp32 training path.  TEST INFRASTRUCTURE ONLY: it is the checker the CUDA
 * library is compared against and the timed CPU baseline; the product
 * (libtenmo_cuda.so and the tenmo_b200 package) never links, imports or calls it.
 *
 * Parity status: the reference is Mojo and cannot be compiled or run where this
 * was written, so the restatement is pinned against the literal known-answer
 * vectors in the reference's own tests (tests/test_mm2d.mojo, test_matmul.mojo,
 * test_mmnd.mojo, test_cross_entropy.mojo, test_sgd.mojo, test_accuracy.mojo ...).
 * Values the reference's tests do not pin (large GEMMs, a full MLP trajectory)
 * are "parity unpinned": they rest on this restatement alone.  exp/log come from
 * libm here and from Mojo's std.math there, so CE results are pinned to ~1 ulp
 * of those functions, not bit-for-bit.
 *
 * All strides and offsets are in ELEMENTS.  All matrices are row-major views
 * (ptr, offset, row_stride, col_stride) exactly like tenmo's NDBuffer.
 */
#ifndef TENMO_REF_H
#define TENMO_REF_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Options shared by the GEMM restatements.
 *  simd_width      : lanes of the reference's SIMD type (8 = AVX2, 16 = AVX-512); decides
 *                    which columns fall into the scalar tail (matmul_cpu.mojo:170-171,337-351).
 *  contract_scalar : 1 = the scalar `acc += a*b` sites are fused multiply-adds,
 *                    0 = separate multiply and add.  Mojo's choice cannot be observed
 *                    without its toolchain, so both are offered.
 *  threads         : worker threads over row tiles (the reference uses num_physical_cores()).
 */
typedef struct {
    int32_t simd_width;
    int32_t contract_scalar;
    int32_t threads;
} tenmo_ref_opts;

typedef struct {
    const float* ptr;
    int64_t offset;
    int64_t row_stride, col_stride;
    int32_t batch_rank;
    int64_t batch_shape[6];
    int64_t batch_stride[6];
} tenmo_ref_mat;

/* MmCpu2d.tiled_matmul + .matmul  (matmul_cpu.mojo:80-135,163-547).  C is (m,p) contiguous. */
void tenmo_ref_matmul_2d(const tenmo_ref_mat* A, const tenmo_ref_mat* B, float* C,
                         int64_t m, int64_t n, int64_t p, const tenmo_ref_opts* opts);

/* MmCpuNd.matmul (matmul_cpu.mojo:627-956): NumPy-style batch broadcast, batch index decoded
 * right to left, an operand's batch stride applied only where its batch dim > 1 (706-724).
 * C is contiguous (total_batch, m, p).  Returns total_batch, or -1 if not broadcastable. */
int64_t tenmo_ref_matmul_nd(const tenmo_ref_mat* A, const tenmo_ref_mat* B, float* C,
                            int64_t m, int64_t n, int64_t p, const tenmo_ref_opts* opts);

/* Naive i-k-j triple loop used by the reference's own tests as their oracle
 * (tests/test_matmul_2d_verify.mojo:8-20). */
void tenmo_ref_matmul_naive(const tenmo_ref_mat* A, const tenmo_ref_mat* B, float* C,
                            int64_t m, int64_t n, int64_t p);

/* out[m,n] = a[m,n] + b[n]  (addition.mojo:71-112 -> cpu_arithmetics.mojo:168-366). */
void tenmo_ref_add_bias(const float* a, const float* b, float* out, int64_t M, int64_t N);
/* out += in, the Gradbox accumulate (ancestry.mojo:83-84 -> gradbox.mojo:1358-1364). */
void tenmo_ref_add_inplace(float* out, const float* in, int64_t n);
/* relu.mojo:97-141: out = max(x,0); mask = x>0 ? 1 : 0. */
void tenmo_ref_relu_fwd(const float* x, float* out, float* mask, int64_t n);
/* relu.mojo:19-46: dx = g * mask. */
void tenmo_ref_relu_bwd(const float* g, const float* mask, float* dx, int64_t n);
/* buffers.mojo:1147-1152: y = 1/(1+exp(-x)). */
void tenmo_ref_sigmoid_fwd(const float* x, float* y, int64_t n);
/* shared/scalar_ops.mojo:131-132 called as out.arithmetic_ops[SIGMOID_BACKWARD](grad): (g*y)*(1-y). */
void tenmo_ref_sigmoid_bwd(const float* g, const float* y, float* dx, int64_t n);
/* Bias gradient: sum over axis 0 of a contiguous (M,N), sequential in m
 * (broadcast.mojo:66-88 -> sum_mean_reduction.mojo:143-156). */
void tenmo_ref_colsum(const float* x, float* out, int64_t M, int64_t N);

/* crossentropy.mojo:285-432 (class-index targets).  reduction: 0 mean, 1 sum, 2 none
 * (shared/__init__.mojo:4-40).  labels are int64.  softmax may be NULL (track_grad=False).
 * loss_out: 1 float (mean/sum) or M floats (none).  Returns valid_count. */
int64_t tenmo_ref_ce_fwd(const float* logits, int64_t stride0, int64_t stride1, const int64_t* labels,
                         int64_t M, int64_t C, int64_t ignore_index, float label_smoothing,
                         int reduction, float* softmax, float* loss_out);
/* crossentropy.mojo:742-766 + 451-481.  upstream: 1 float (mean/sum) or M floats (none). */
void tenmo_ref_ce_bwd(const float* softmax, const int64_t* labels, int64_t M, int64_t C,
                      int64_t ignore_index, float label_smoothing, int reduction,
                      const float* upstream, int64_t valid_count, float* dlogits);

/* optim.mojo:123-158 (momentum) and 100-121 (plain).  momentum == 0 selects the plain form,
 * as SGD.step does. */
void tenmo_ref_sgd_step(float* p, const float* g, float* v, int64_t n, float lr, float momentum,
                        float weight_decay);

/* accuracy.mojo:20-66: first-index argmax (strict >), count of rows equal to the label. */
int64_t tenmo_ref_accuracy(const float* logits, int64_t s0, int64_t s1, const int64_t* labels,
                           int64_t M, int64_t C);

/* One MLP training step through the restated Linear/ReLU/CE/backward/SGD sequence
 * (net.mojo:179-216, relu.mojo, crossentropy.mojo, matmul.mojo:24-54, broadcast.mojo:66-88,
 * optim.mojo:405-543).  dims has n_layers+1 entries; W[l] is (dims[l], dims[l+1]) row-major;
 * ReLU after every layer but the last.  Returns the mean loss; if logits_out != NULL the
 * forward logits (batch, dims[n_layers]) are copied there.  grads (dW, db) are left in
 * dW[l], db[l] when those are non-NULL.  grad_scale multiplies the gradients before the
 * update (1/world for data parallel).  do_update == 0 skips SGD. */
float tenmo_ref_mlp_step(int n_layers, const int64_t* dims, float** W, float** b, float** vW, float** vb,
                         float** dW, float** db,
                         const float* X, const int64_t* labels, int64_t batch,
                         float lr, float momentum, float weight_decay, float grad_scale, int do_update,
                         float* logits_out, const tenmo_ref_opts* opts);

/* Conv2d on a PRE-PADDED image, NCHW (cnn.mojo:404-507): per output, the accumulator starts at the bias and
 * adds img * kernel over (c_in, ky, kx) ascending.  contract = 1 fuses each multiply-add. */
void tenmo_ref_conv2d_fwd(const float* img, const float* kernel, const float* bias, float* out, int64_t N, int64_t Cin,
                          int64_t Hp, int64_t Wp, int64_t Cout, int KH, int KW, int stride, int dilation, int contract);
/* Gradients of the same op (cnn.mojo:664-950): db per-channel sum, dW = grad (C_out, N*Ho*Wo) . patches,
 * dX scatter of kernel-weighted gradients.  Any of d_img / d_kernel / d_bias may be NULL. */
void tenmo_ref_conv2d_bwd(const float* grad, const float* img, const float* kernel, float* d_img, float* d_kernel,
                          float* d_bias, int64_t N, int64_t Cin, int64_t Hp, int64_t Wp, int64_t Cout, int KH, int KW,
                          int stride, int dilation);
/* MaxPool2d (pooling.mojo:301-402, 25-107): k x k window walked row by row, strict >, argmax = y*W + x or -1. */
void tenmo_ref_maxpool2d_fwd(const float* x, float* out, int64_t* argmax, int64_t NC, int64_t H, int64_t W, int k, int stride,
                             int pad);
void tenmo_ref_maxpool2d_bwd(const float* g, const int64_t* argmax, float* dx, int64_t NC, int64_t H, int64_t W, int64_t Ho,
                             int64_t Wo);

/* Softmax over the last axis of a contiguous (M, C) matrix (softmax.mojo:30-48,165-178; row sums in the chunked
 * order of buffers.mojo:1304-1333 with simd_width lanes) and its backward y * (g - sum(g * y)) (softmax.mojo:206-213). */
void tenmo_ref_softmax_fwd(const float* x, float* y, int64_t M, int64_t C, int simd_width);
void tenmo_ref_softmax_bwd(const float* g, const float* y, float* dx, int64_t M, int64_t C, int simd_width);

/* M[m,k] @ v[k] (matrixvector.mojo:269-282) and v[k] @ M[k,n] (vectormatrix.mojo:283-340): one ascending
 * accumulation chain per output; strides in elements; contract as in tenmo_ref_opts. */
void tenmo_ref_mv(const float* M, int64_t m_s0, int64_t m_s1, const float* v, int64_t v_s, float* out, int64_t m,
                  int64_t k, int contract);
void tenmo_ref_vm(const float* v, int64_t v_s, const float* M, int64_t m_s0, int64_t m_s1, float* out, int64_t k,
                  int64_t n, int contract);

#ifdef __cplusplus
}
#endif
#endif
