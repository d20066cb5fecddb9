/*
 * C ABI of the B200 (sm_100a) implementation of portDNN's convolution hot path.
 *
 * portDNN itself exposes no C ABI: its boundary is the set of C++ launch templates in
 * include/portdnn/<op>/launch.h, which forward to SNN_EXPORT'ed template instantiations
 * inside libportdnn.so (e.g. internal::launch_direct, include/portdnn/internal/conv2d/direct.h:34-39).
 * Every entry point below replaces one such exported launcher; the C++ headers under
 * include/portdnn/ rebuild the reference's templates on top of these functions.
 *
 * Conventions
 *  - All pointers are device pointers unless stated; the caller owns every buffer.
 *  - All work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default
 *    stream) and the call returns without synchronising.
 *  - Return value: a PdnnStatus with the numeric values of sycldnn::StatusCode
 *    (include/portdnn/status.h:31-44). Nothing throws. There is no CPU fallback: without a
 *    CUDA device every compute entry point returns PDNN_ALLOCATION_PROBLEM.
 *  - dtype selects the element type of every tensor of the call: fp32 tensors are multiplied
 *    with a 3xTF32 split on the tensor cores (or fp32 FMA in the direct kernels); fp16/bf16
 *    tensors accumulate in fp32.
 */
#ifndef PORTDNN_B200_H_
#define PORTDNN_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* sycldnn::StatusCode, include/portdnn/status.h:31-44 */
typedef enum PdnnStatus {
  PDNN_OK = 0,
  PDNN_INVALID_ALGORITHM = 1,
  PDNN_INDEX_EXCEEDED = 2,
  PDNN_INSUFFICIENT_WORKSPACE = 3,
  PDNN_ALLOCATION_PROBLEM = 4,
  PDNN_INVALID_PARAMETER = 5
} PdnnStatus;

typedef enum PdnnDataType { PDNN_F32 = 0, PDNN_F16 = 1, PDNN_BF16 = 2 } PdnnDataType;

/* sycldnn::conv2d::conv_type::{Forward,InputBackprop,FilterBackprop}, include/portdnn/conv2d/conv_type.h:32-48 */
typedef enum PdnnPass { PDNN_FORWARD = 0, PDNN_INPUT_BACKPROP = 1, PDNN_FILTER_BACKPROP = 2 } PdnnPass;

/* sycldnn::conv2d::Algorithm, include/portdnn/conv2d/algorithm.h:30-45.  Direct runs the
 * general SIMT kernel; Tiled, Im2col and Matmul run the tcgen05 implicit-GEMM kernel (which
 * needs no im2col buffer); Winograd and WinogradLarge run Winograd F(2x2,3x3) (transforms around
 * a batched tcgen05 matmul) on 3x3 stride-1 forward / input-backprop layers when the caller
 * passes the workspace pdnn_conv2d_workspace_size recommends, and the implicit-GEMM kernel
 * otherwise.  A shape the tensor-core kernels cannot take
 * (channel or feature count not a multiple of 8 elements of 16 bits / 4 of 32 bits) is routed
 * to the direct kernel whatever the algorithm. */
typedef enum PdnnAlgorithm {
  PDNN_ALGO_NOT_SUPPORTED = 0,
  PDNN_ALGO_DIRECT = 1,
  PDNN_ALGO_TILED = 2,
  PDNN_ALGO_IM2COL = 3,
  PDNN_ALGO_WINOGRAD = 4,
  PDNN_ALGO_WINOGRAD_LARGE = 5,
  PDNN_ALGO_MATMUL = 6
} PdnnAlgorithm;

/* sycldnn::pooling::{Max,MaxWithNan,Average}, include/portdnn/pooling/operators.h */
typedef enum PdnnPoolOp { PDNN_POOL_MAX = 0, PDNN_POOL_MAX_WITH_NAN = 1, PDNN_POOL_AVERAGE = 2 } PdnnPoolOp;

/* sycldnn::pointwise::{Relu,Tanh}, include/portdnn/pointwise/operators.h.  PDNN_ACT_RELU6 has no
 * counterpart in the reference (min(max(x,0),6)); it exists for the MobileNet-v2 workload. */
typedef enum PdnnActivation { PDNN_ACT_NONE = -1, PDNN_ACT_RELU = 0, PDNN_ACT_TANH = 1, PDNN_ACT_RELU6 = 2 } PdnnActivation;
/* The remaining sycldnn::pointwise operators (Exp, Log, Floor, Sqrt): accepted by pdnn_pointwise
 * and, except Floor, pdnn_pointwise_grad, which take either enum; not valid as a fused activation. */
typedef enum PdnnPointwiseOp { PDNN_PW_EXP = 3, PDNN_PW_LOG = 4, PDNN_PW_FLOOR = 5, PDNN_PW_SQRT = 6 } PdnnPointwiseOp;

/* Field-for-field mirror of sycldnn::conv2d::Conv2DParams (include/portdnn/conv2d/params.h:32-112).
 * input_format: 0 NHWC, 1 NCHW (include/portdnn/data_format.h:31-43); filter_format: 0 HWCF, 1 FCHW,
 * 2 FHWC (include/portdnn/filter_format.h:32-53); group_format: 0 STRIDED, 1 INTERLEAVED. */
typedef struct PdnnConv2DParams {
  int channels, features, batch, in_rows, in_cols;
  int window_rows, window_cols, stride_rows, stride_cols;
  int out_rows, out_cols, pad_rows, pad_cols;
  int dilation_rows, dilation_cols, groups;
  int input_format, filter_format, group_format;
} PdnnConv2DParams;

/* Mirror of sycldnn::depthwise_conv2d::DepthwiseConv2DParams (include/portdnn/depthwise_conv2d/params.h:33-94). */
typedef struct PdnnDepthwiseConv2DParams {
  int channels, channel_multiplier, batch, in_rows, in_cols;
  int window_rows, window_cols, stride_rows, stride_cols;
  int out_rows, out_cols, pad_rows, pad_cols;
} PdnnDepthwiseConv2DParams;

/* Mirror of sycldnn::pooling::PoolingParams (include/portdnn/pooling/params.h:30-73). */
typedef struct PdnnPoolingParams {
  int in_rows, in_cols, out_rows, out_cols;
  int window_rows, window_cols, stride_rows, stride_cols;
  int batch, channels, pad_rows, pad_cols;
  int input_format;
} PdnnPoolingParams;

/* Mirror of sycldnn::softmax::SoftmaxParams (include/portdnn/softmax/params.h:27-54). */
typedef struct PdnnSoftmaxParams {
  int channels, batch, rows, cols;
  int input_format; /* 0 = NHWC (the only layout implemented) */
} PdnnSoftmaxParams;

/* Mirror of sycldnn::batchnorm::BatchNormParams (include/portdnn/batchnorm/params.h:32-72). */
typedef struct PdnnBatchNormParams {
  int batch, rows, cols, channels;
  int is_training; /* 0: frozen (population statistics handed in), 1: training */
  float epsilon, momentum;
  int input_format; /* 0 = NHWC (the only layout implemented) */
} PdnnBatchNormParams;

/* Optional fused epilogue of the forward convolution: out = act(alpha*conv + bias[k]) + beta*out_prev.
 * The reference has no fused form: it issues binaryop Add (tools/layer.h:100-125), a pointwise
 * launch (tools/layer.h:207-228) and the compat alpha/beta blend (include/portdnn/compat/scaling.hpp:202-281)
 * as separate kernels; the fused result matches that chain. bias may be NULL. */
typedef struct PdnnConvEpilogue {
  const void* bias;  /* [features], same dtype as the tensors; NULL = none */
  int activation;    /* PdnnActivation */
  float alpha;       /* scales the convolution result; 1 = plain */
  float beta;        /* scales the previous contents of out; 0 = overwrite */
  void* relu_bitmask; /* optional second output (NULL = none), NHWC with features % 8 == 0: one bit per
                         output element, bit (i % 8) of byte (i / 8) for element i, set where the result is
                         positive - the ReLU mask a later input backprop needs, at a sixteenth of the bytes
                         (PdnnBackpropFusion::relu_bitmask) */
  int constant_filter; /* non-zero: the caller states that filter and bias were not written by the kernel that
                          precedes this call in the stream (the weights of a trained network).  The
                          convolution kernel is launched so that its set-up overlaps the end of that kernel
                          (programmatic dependent launch) and then waits for it before it touches a tensor;
                          with this flag it fetches the filter and the bias before that wait.  0 is always safe. */
} PdnnConvEpilogue;

/* Replaces conv2d::launch -> sublaunch -> launch_{direct,tiled,im2col,winograd,matmul}
 * (include/portdnn/conv2d/launch.h:59-118, include/portdnn/internal/conv2d/launch.h:169-207).
 * Argument slots as in the reference: Forward (x, w, y); InputBackprop (dy, w, dx);
 * FilterBackprop (x, dy, dW).  workspace_elems counts ELEMENTS of dtype, as
 * query_workspace_size does (include/portdnn/conv2d/workspace_size.h:42-47). When the chosen
 * kernel needs scratch and workspace is NULL or too small the library takes it from the
 * stream-ordered allocator (cudaMallocAsync) for the duration of the call, the way the
 * reference's im2col driver self-allocates (include/portdnn/internal/conv2d/im2col.h:224-246). */
int pdnn_conv2d(int pass, int dtype, const void* input, const void* filter, void* output,
                const PdnnConv2DParams* params, int algorithm, void* workspace, size_t workspace_elems,
                void* stream);

/* As pdnn_conv2d for PDNN_FORWARD, with the fused epilogue described at PdnnConvEpilogue. */
int pdnn_conv2d_fused(int dtype, const void* input, const void* filter, void* output,
                      const PdnnConv2DParams* params, int algorithm, const PdnnConvEpilogue* epilogue,
                      void* workspace, size_t workspace_elems, void* stream);

/* Optional fused forms of the two backprop passes.  The reference has none: a training step built
 * on it runs pointwise::launch<Relu, Gradient> (include/portdnn/pointwise/launch.h:133-179) on every
 * activation gradient and keeps filter gradients in the tensors' own type; the fused results match
 * that chain.
 *  - relu_forward_output (InputBackprop only; NULL = none): the forward output y_prev of the layer
 *    whose ReLU precedes this convolution, same shape as dx.  The call returns
 *    dx[i] = y_prev[i] > 0 ? dx[i] : 0, i.e. the gradient with respect to that layer's
 *    pre-activation, which is what its own two backprop passes consume.
 *  - output_f32 (FilterBackprop only): dW is written as fp32 even for fp16 / bf16 tensors, so that
 *    it can land directly in the fp32 buffer a gradient all-reduce works on.
 *  - accumulate: InputBackprop: dx already holds the gradient that arrived through another
 *    reader of the tensor (a shortcut branch); this call adds its own to it, dx += conv_backprop(dy, w),
 *    and the mask of relu_forward_output, when given, applies to the sum - the reference chain of
 *    an input backprop into a temporary, binaryop::launch<Add> and the ReLU gradient.  The value 2
 *    says that dx already carries that mask (every earlier contribution applied it): the result is
 *    the same, but positions a strided convolution does not reach are left untouched instead of
 *    being read, masked and written again.
 *    FilterBackprop: dW += gradient (gradient accumulation over micro-batches, or into a buffer the
 *    caller zeroed).  With fp32 gradients the pixel splits of the kernel add their tiles to dW
 *    directly (TMA reduction) instead of writing partial sums for a second kernel, so no workspace
 *    is used and the order of the float additions is not fixed from run to run.
 *  - relu_bitmask (InputBackprop only, 16-bit tensors, channels % 8 == 0): the same mask as
 *    relu_forward_output > 0 in the one-bit-per-element form PdnnConvEpilogue::relu_bitmask writes;
 *    give one or the other. */
typedef struct PdnnBackpropFusion {
  const void* relu_forward_output;
  int output_f32;
  int accumulate;
  const void* relu_bitmask;
  int constant_filter; /* InputBackprop: as PdnnConvEpilogue::constant_filter, for the filter */
} PdnnBackpropFusion;

/* As pdnn_conv2d for PDNN_INPUT_BACKPROP / PDNN_FILTER_BACKPROP, with the fused forms described at
 * PdnnBackpropFusion (fusion == NULL: exactly pdnn_conv2d). */
int pdnn_conv2d_backprop_fused(int pass, int dtype, const void* input, const void* filter, void* output,
                               const PdnnConv2DParams* params, int algorithm, const PdnnBackpropFusion* fusion,
                               void* workspace, size_t workspace_elems, void* stream);

/* Replaces conv2d::query_workspace_size (include/portdnn/conv2d/workspace_size.h:158-163). Sizes in elements. */
int pdnn_conv2d_workspace_size(int pass, int dtype, const PdnnConv2DParams* params, int algorithm,
                               size_t* required_elems, size_t* recommended_elems);

/* Parameter checks of conv2d::validate_params + sublaunch (include/portdnn/internal/conv2d/launch.h:42-97,169-197)
 * without launching anything; host only. */
int pdnn_conv2d_validate(int pass, const PdnnConv2DParams* params, int algorithm);

/* Replaces depthwise_conv2d::launch (include/portdnn/depthwise_conv2d/launch.h:54-91,
 * src/depthwise_conv2d/launch.cc:41-121).  Filter is [R][S][C][mult]; slots as for pdnn_conv2d.
 * The filter-backprop pass reduces over batch and image in two stages and needs
 * pdnn_depthwise_workspace_bytes() of scratch; with workspace NULL it is taken from the
 * stream-ordered allocator. */
int pdnn_depthwise_conv2d(int pass, int dtype, const void* input, const void* filter, void* output,
                          const PdnnDepthwiseConv2DParams* params, void* workspace, size_t workspace_bytes,
                          void* stream);
size_t pdnn_depthwise_workspace_bytes(int pass, int dtype, const PdnnDepthwiseConv2DParams* params);

/* No counterpart in the reference.  The filter-backprop pass of pdnn_depthwise_conv2d for hosts
 * that may not allocate device memory once they are running - an inference server with a fixed
 * memory plan, a framework that owns the whole device heap, a latency-critical loop where an
 * allocator call is not allowed.  Same arguments, same result: (x, dy) -> dW for the filter
 * [R][S][C][mult].  The partial sums live in one fixed 8 MiB array inside the library
 * (pdnn_noalloc_scratch_bytes()); the call performs no cudaMalloc, cudaFree or other allocating
 * call.  It returns PDNN_INSUFFICIENT_WORKSPACE when R*S*C*mult*4 bytes exceed that array.
 *  - The first call on each device looks the array's device address up (a one-time, host-side
 *    query made with that device current); make that first call before any stream capture.
 *  - All calls on a device share the array, and it keeps whatever the last call left there.
 *    Every call overwrites the part it reads, so stale contents never reach a result, but two
 *    calls that overlap on the GPU (different streams, no ordering between them) race on it:
 *    keep calls to this entry point ordered. */
int pdnn_depthwise_filter_backprop_noalloc(int dtype, const void* input, const void* output_grad, void* filter_grad,
                                           const PdnnDepthwiseConv2DParams* params, void* stream);
size_t pdnn_noalloc_scratch_bytes(void);

/* Replaces pooling::launch, two-pointer form (include/portdnn/pooling/launch.h:112-180,
 * src/pooling/launch_pooling.cc:89-165): forward for every op (input -> output) and the
 * average gradient (direction 1: input = dy, output = dx).  input_format 1 (NCHW) runs the NHWC
 * kernel between two transposes in scratch from the stream-ordered allocator. */
int pdnn_pooling(int op, int direction, int dtype, const void* input, void* output,
                 const PdnnPoolingParams* params, void* stream);

/* Replaces pooling::launch, four-pointer form for the max gradient
 * (include/portdnn/pooling/launch.h:182-257): (x, y, dy) -> dx. */
int pdnn_pooling_max_grad(int op, int dtype, const void* input_data, const void* output_data,
                          const void* input_backprop, void* output_backprop,
                          const PdnnPoolingParams* params, void* stream);

/* The same followed by pointwise::launch<Relu, Gradient> with input_data as the forward tensor, in one
 * call (no reference counterpart): for a pooled tensor that is the output of a ReLU, output_backprop is
 * the gradient with respect to that ReLU's input, i.e. elements of input_data that are not positive
 * receive nothing.  For 3x3 windows it costs nothing extra: a window whose maximum is not positive
 * simply has no winner. */
int pdnn_pooling_max_grad_relu(int op, int dtype, const void* input_data, const void* output_data,
                               const void* input_backprop, void* output_backprop,
                               const PdnnPoolingParams* params, void* stream);

/* Replaces softmax::launch<T, Forward / Gradient> (include/portdnn/softmax/launch.h:64-165):
 * y = exp(x - max) / sum exp(x - max) over the channels of each pixel.  direction 0: input = x,
 * gradient unused.  direction 1: input = the forward OUTPUT y, gradient = dy,
 * output = (dy - sum_c(dy * y)) * y.  No workspace is needed (the reference's is ignored). */
int pdnn_softmax(int direction, int dtype, const void* input, const void* gradient, void* output,
                 const PdnnSoftmaxParams* params, void* stream);

/* Replaces batchnorm::launch<T, Backend, Forward> (include/portdnn/batchnorm/launch.h:222-330).
 * output = (x - mean) / sqrt(variance + eps) * gamma + beta with the mean and variance HANDED IN,
 * in both modes (include/portdnn/internal/batchnorm/launch_internal.h:95-158).  Training
 * additionally writes running_mean = batch_mean * (1 - momentum) + mean * momentum and
 * running_variance likewise from the biased batch variance; frozen ignores the running pointers. */
int pdnn_batchnorm_forward(int dtype, const void* input, const void* beta, const void* gamma, const void* mean,
                           const void* variance, void* running_mean, void* running_variance, void* output,
                           const PdnnBatchNormParams* params, void* stream);

/* Replaces batchnorm::launch<T, Backend, Gradient> (include/portdnn/batchnorm/launch.h:332-444):
 * input gradient, beta gradient (sum dy) and gamma gradient.  Training uses the batch statistics
 * of `input`; frozen uses pop_mean / pop_variance (ignored when training)
 * (launch_internal.h:318-640). */
int pdnn_batchnorm_gradient(int dtype, const void* input, const void* gradient, const void* gamma,
                            const void* pop_mean, const void* pop_variance, void* beta_grad, void* gamma_grad,
                            void* output, const PdnnBatchNormParams* params, void* stream);

/* Replaces pointwise::launch forward / gradient (include/portdnn/pointwise/launch.h:61-179); op is
 * a PdnnActivation (not NONE) or a PdnnPointwiseOp.  The gradient's first tensor is the forward
 * OUTPUT, as the reference kernel treats it (src/pointwise/kernels.h:205-233); Floor has no
 * gradient (InvalidParameter), and Exp's is the reference's exp(v) + err (kernels.h:94-101). */
int pdnn_pointwise(int op, int dtype, const void* input, void* output, size_t n_items, void* stream);
int pdnn_pointwise_grad(int op, int dtype, const void* output_forward, const void* input_backprop,
                        void* output_backprop, size_t n_items, void* stream);

/* Replaces binaryop::launch<Add> in its bias form, lhs_dims={rows,C}, rhs_dims={1,C}
 * (include/portdnn/binaryop/launch.h:58-97, test/bias/bias_fixture.h:78-85), optionally followed
 * by an activation in the same pass (PDNN_ACT_NONE for the plain reference behaviour). */
int pdnn_bias_add(int dtype, const void* input, const void* bias, void* output, size_t rows, int channels,
                  int activation, void* stream);

/* Replaces binaryop::launch<T, Op> (include/portdnn/binaryop/launch.h:58-97, operators.h:29-35):
 * output = lhs (op) rhs with numpy-style broadcasting.  Each operand has at most four extents
 * (binaryop/params.h:31), none (n == 0) meaning a scalar; the shorter shape is padded with leading
 * ones, each pair of extents must be equal or hold a one, the output takes the larger of each
 * pair (include/portdnn/internal/binaryop/launch.h:34-57).  InvalidParameter otherwise. */
typedef enum PdnnBinaryOp { PDNN_BINARY_ADD = 0, PDNN_BINARY_SUB = 1, PDNN_BINARY_MUL = 2, PDNN_BINARY_DIV = 3 } PdnnBinaryOp;
int pdnn_binaryop(int op, int dtype, const void* lhs, const int* lhs_dims, int n_lhs_dims, const void* rhs,
                  const int* rhs_dims, int n_rhs_dims, void* output, void* stream);

/* out = alpha*a + beta*b elementwise (b may be NULL when beta == 0): the compat layer's
 * alpha/beta blend, include/portdnn/compat/scaling.hpp:202-281, as one pass. */
int pdnn_scale_blend(int dtype, const void* a, float alpha, const void* b, float beta, void* out, size_t n_items,
                     void* stream);

/* Replaces transpose::launch and convert_nhwc_to_nchw / convert_nchw_to_nhwc
 * (include/portdnn/transpose/launch.h:66-233): output extent d is dims[permutation[d]] and
 * out[i_permutation[0]][i_permutation[1]]... = in[i_0][i_1]...  Elements are moved as raw words of
 * elem_bytes (1, 2, 4 or 8) bytes, as the reference does (include/portdnn/internal/transpose/launch.h:47-83);
 * up to six dimensions; not in place. */
int pdnn_transpose(int elem_bytes, const void* input, void* output, const int* dims, int n_dims, const int* permutation,
                   void* stream);

/* Replaces matmul::launch / Backend::matmul / Backend::batch_matmul
 * (include/portdnn/matmul/launch.h:37-90, include/portdnn/backend/backend_interface.h:78-118):
 * out[b] = beta*out[b] + op(lhs[b]) * op(rhs[b]), row-major, strided batches. */
int pdnn_matmul(int dtype, int transpose_lhs, int transpose_rhs, const void* lhs, const void* rhs, void* output,
                int batches, int m, int k, int n, float beta, void* stream);

/* The collective of the batch-sharded path; no counterpart in the reference, which is single-device.
 * Each rank's filter-backprop pass leaves fp32 gradients for its shard of the batch in one contiguous
 * buffer; pdnn_allreduce_filter_grads sums `count` floats of it over the ranks in place with
 * ncclAllReduce on `stream` (any sub-range of the buffer may be reduced on its own, so a caller can
 * start a stage's reduction while the backward pass continues on another stream).
 * pdnn_comm_unique_id fills 128 bytes on rank 0; every rank passes the same bytes to pdnn_comm_init
 * with its CUDA device current.  NCCL is looked up in the process at the first call
 * (PDNN_ALLOCATION_PROBLEM if libnccl.so.2 cannot be found). */
int pdnn_comm_unique_id(void* id128);
int pdnn_comm_init(void** comm, const void* id128, int world_size, int rank);
int pdnn_allreduce_filter_grads(void* comm, float* gradients, size_t count, void* stream);
int pdnn_comm_destroy(void* comm);

/* Reads (and optionally clears) the 4-word record the tensor-core kernels fill when one of
 * their bounded waits gives up instead of spinning: word 0 is 0 when nothing went wrong, else
 * 1 (wait timed out), word 1 the CTA, word 2 the wait site, word 3 the phase parity.
 * Synchronises the device.  The reference has no counterpart (its kernels never wait on one
 * another). */
int pdnn_device_error_record(unsigned words[4], int clear);

/* Text of the last failure recorded by this thread ("" if none); host only. */
const char* pdnn_last_error(void);

/* Number of kernels this library has launched in the calling process; host only. */
unsigned long long pdnn_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* PORTDNN_B200_H_ */
