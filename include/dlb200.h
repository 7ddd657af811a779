/* dlb200 — B200 (sm_100a) kernels for the fully-connected training step of the
 * SebastienKeroack/deep-learning library, behind a C ABI.
 *
 * Every entry point takes plain pointers and sizes.  Device pointers are
 * ordinary CUDA device addresses owned by the caller (or obtained from
 * dlb_malloc); all work is enqueued on the context's stream and nothing blocks
 * the host except dlb_ctx_sync, dlb_memcpy_d2h and the functions documented as
 * synchronous.  No function throws; each returns a dlb_status.
 *
 * Layouts are the reference's: activations are row-major [rows, units] per time
 * step, weights of a layer are row-major [units_out, units_in], and the flat
 * parameter vector is { all W | all bias | all gamma | all beta }
 * (lib/deep-learning/v1/learner/compile.cpp L:610-695,
 *  connections_prepare.cpp L:21-81, allocate.cpp L:1150-1233).
 *
 * Citations "ref:" name the reference function each entry point replaces, by
 * path inside the reference project.
 */
#ifndef DLB200_H_
#define DLB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int dlb_status;
enum {
  DLB_OK = 0,
  DLB_ERR_INVALID = 1,      /* bad argument (null pointer, size, enum) */
  DLB_ERR_CUDA = 2,         /* a CUDA runtime/driver call failed */
  DLB_ERR_UNSUPPORTED = 3,  /* combination outside the supported path */
  DLB_ERR_TIMEOUT = 4,      /* a bounded device-side wait gave up */
  DLB_ERR_COMM = 5,         /* NCCL error */
  DLB_ERR_NO_DEVICE = 6     /* no sm_100 device: there is no CPU fallback */
};

/* Numeric values of the reference's enums (v1/data/enum/*.hpp). */
enum { DLB_AF_ELU = 3, DLB_AF_ISRLU = 10, DLB_AF_LINEAR = 11, DLB_AF_LEAKY_RELU = 14,
       DLB_AF_RELU = 16, DLB_AF_SELU = 17, DLB_AF_SOFTMAX = 22 };
enum { DLB_DROPOUT_NONE = 0, DLB_DROPOUT_BERNOULLI = 2, DLB_DROPOUT_BERNOULLI_INVERTED = 3,
       DLB_DROPOUT_SHAKEDROP = 5, DLB_DROPOUT_UOUT = 6 };
enum { DLB_OPT_ADABOUND = 1, DLB_OPT_ADAM = 2, DLB_OPT_ADAMAX = 3, DLB_OPT_AMSBOUND = 4,
       DLB_OPT_AMSGRAD = 5, DLB_OPT_GD = 6, DLB_OPT_NOSADAM = 9 };
enum { DLB_LOSS_CROSS_ENTROPY = 2, DLB_LOSS_MSE = 10 };
enum { DLB_LAYER_FULLY_CONNECTED = 3, DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT = 4,
       DLB_LAYER_LSTM = 7, DLB_LAYER_RESIDUAL = 9 };
enum { DLB_NORM_NONE = 0, DLB_NORM_BATCH_NORMALIZATION = 1, DLB_NORM_BATCH_RENORMALIZATION = 2 };
enum { DLB_MODEL_FEEDFORWARD = 3, DLB_MODEL_RECURRENT = 4 };
enum { DLB_PROPAGATION_INFERENCE = 0, DLB_PROPAGATION_TRAINING = 1 };
enum { DLB_ACCU_CROSS_ENTROPY = 1, DLB_ACCU_DISTANCE = 3 };

const char *dlb_status_string(dlb_status s);
/* Last error text recorded on the calling thread ("" if none). */
const char *dlb_last_error(void);
int dlb_version(void);

/* ------------------------------------------------------------------------ */
/* Context: one per GPU, single caller at a time (the reference's step
 * functions are likewise entered by one OpenMP team, drivers/driver.cpp
 * L:241-257).  Owns a stream, a scratch arena for reduction partials and
 * TF32 residual planes, and optionally an NCCL communicator. */
typedef struct dlb_ctx dlb_ctx;

dlb_status dlb_ctx_create(dlb_ctx **out, int device);
dlb_status dlb_ctx_destroy(dlb_ctx *ctx);
/* Waits for the stream; *device_status receives the sticky device status word
 * (DLB_OK, or DLB_ERR_TIMEOUT if a kernel's bounded wait expired). */
dlb_status dlb_ctx_sync(dlb_ctx *ctx, int *device_status);
void *dlb_ctx_stream(dlb_ctx *ctx); /* cudaStream_t */
/* 0: always the CUDA-core GEMM; 1 (default): tcgen05 GEMM when shapes allow. */
dlb_status dlb_ctx_set_tensor_core(dlb_ctx *ctx, int enable);
/* Number of kernels this context has launched since creation. */
uint64_t dlb_ctx_launch_count(dlb_ctx *ctx);
/* Device-side timing on the context's stream (CUDA events): start records an
 * event, stop records another, waits for it and returns the milliseconds
 * between the two. */
dlb_status dlb_ctx_timer_start(dlb_ctx *ctx);
dlb_status dlb_ctx_timer_stop(dlb_ctx *ctx, float *milliseconds);
/* Per-launch timing of the tensor-core GEMM: while enabled every launch is
 * bracketed by a pair of events.  dlb_ctx_gemm_profile_read waits for the
 * stream, returns the number of launches, their summed duration and their
 * summed algorithmic FLOPs (2*M*N*K each, not multiplied by the three
 * tensor-core products issued per FLOP), and clears the record. */
dlb_status dlb_ctx_gemm_profile(dlb_ctx *ctx, int enable);
dlb_status dlb_ctx_gemm_profile_read(dlb_ctx *ctx, uint64_t *launches, double *milliseconds,
                                     double *flops);
/* While the same profiling is on, two more things are bracketed by events on the
 * context's stream: every wait of the stream for the overlapped gradient
 * all-reduces (dlb_comm_join: the part of the transfers that the kernels did
 * not hide) and every exchange of batch-renormalization sums
 * (dlb_allreduce_f64).  Their counts and summed durations over the records that
 * the last dlb_ctx_gemm_profile_read consumed: */
dlb_status dlb_ctx_comm_profile_read(dlb_ctx *ctx, uint64_t *join_waits, double *join_wait_ms,
                                     uint64_t *exchanges, double *exchange_ms);

/* Device memory for callers without their own CUDA binding. */
dlb_status dlb_malloc(dlb_ctx *ctx, void **dev_ptr, size_t bytes);
dlb_status dlb_free(dlb_ctx *ctx, void *dev_ptr);
dlb_status dlb_memset(dlb_ctx *ctx, void *dev_ptr, int value, size_t bytes);
dlb_status dlb_memcpy_h2d(dlb_ctx *ctx, void *dev_dst, const void *host_src, size_t bytes);
/* Synchronous: returns after the bytes are in host memory. */
dlb_status dlb_memcpy_d2h(dlb_ctx *ctx, void *host_dst, const void *dev_src, size_t bytes);
dlb_status dlb_memcpy_d2d(dlb_ctx *ctx, void *dev_dst, const void *dev_src, size_t bytes);
/* Free and total bytes of the current device (cudaMemGetInfo), for callers that
 * watch what the library allocates. */
dlb_status dlb_device_mem_info(size_t *free_bytes, size_t *total_bytes);
/* Pinned host memory for staging inputs. */
dlb_status dlb_host_alloc(void **host_ptr, size_t bytes);
dlb_status dlb_host_free(void *host_ptr);

/* ------------------------------------------------------------------------ */
/* TF32 residual plane.  The tensor-core GEMMs compute a*b as
 * hi(a)*hi(b) + hi(a)*lo(b) + lo(a)*hi(b) ("3xTF32"), where hi(x) is what the
 * tensor core sees of the fp32 word x (its top 19 bits) and lo(x) is the
 * exactly representable remainder x - hi(x), rounded to TF32.  A `_lo`
 * argument is a caller-kept plane of those remainders with the shape of its
 * tensor; pass NULL and the library derives it into context scratch first. */
dlb_status dlb_split_tf32(dlb_ctx *ctx, const float *x, float *x_lo, size_t n);

/* The same product on fp16 tensor-core inputs ("3xFP16", the default): every
 * operand tensor x is scaled by a power of two s chosen from max |x| so that
 * s*max lies in [2^14, 2^15), and used as hi = fp16(s x), lo = fp16(s x - hi):
 * 22 bits of every element that is within 2^-17 of the tensor's largest, an
 * absolute floor of 2^-39 max below that.  The three products hi*hi, hi*lo,
 * lo*hi run at twice the TF32 rate and are exact in the fp32 accumulator; the
 * result is scaled back by 1 / (s_a s_b), exactly.
 *
 * Under this form the `_lo` argument of an entry point is the tensor's plane
 * buffer: storage of the tensor's own byte size (n floats) that dlb_split_planes
 * fills with the two fp16 planes, remembering the tensor, its size and the
 * device slot of s under the buffer's address.  Entry points that produce an
 * operand tensor and take a `_lo` output (dlb_activation_forward,
 * dlb_brn_backward_apply, dlb_loss_delta, ...) fill it in whichever form the
 * context is in, so a caller's code is the same for both.  A `_lo` pointer that
 * was not written that way is ignored and the planes are derived per call. */
enum { DLB_GEMM_TF32X3 = 0, DLB_GEMM_F16X3 = 1 };
dlb_status dlb_ctx_set_gemm_kind(dlb_ctx *ctx, int kind);
int dlb_ctx_gemm_kind(dlb_ctx *ctx);
/* Plane buffer of x in the context's current form (TF32: dlb_split_tf32). */
dlb_status dlb_split_planes(dlb_ctx *ctx, const float *x, float *planes, size_t n);
/* The same for a row-major [rows, cols] tensor.  Knowing the shape, the split
 * also records the largest |x| of every row and every column for the range
 * guard of the fp16 form: the planes carry 22 bits of an element only while
 * it is within 2^-17 of the tensor's largest, so a row or column whose every
 * element is far smaller than the rest of the tensor would come out of a
 * product with less than fp32 accuracy relative to its own size.  Such a tensor
 * is flagged: rows and columns separately (a non-zero maximum below 2^-21 of
 * the tensor's), and as a whole when it holds NaN or infinity or, in a
 * stand-alone split, a value that overflows the scale.  A small line
 * only costs accuracy where it is a line of the product's output, i.e. along
 * the operand's free dimension; along the contraction its terms are added to
 * those of the large lines.  The tensor-core kernel therefore skips a product
 * when an operand overflowed or has small lines along its free dimension, and an
 * fp32 CUDA-core kernel computes that product instead.  dlb_ctx_guard_counters
 * reads how often that happened: operand tensors flagged, products that took the
 * fp32 kernel.  Entry points that produce an operand tensor together with its
 * plane buffer record the same statistics.  The check sees each operand alone: a
 * column that is small in one operand and made up for by a huge column in the
 * other is not detected; the TF32 form has fp32 range throughout.
 *
 * Inside a model (dlb_model_*) the errors of the backward pass are exempt from
 * the row flag: their rows are the examples of the batch, and after a few steps
 * of a classifier most of them are 2^-20 and less of the few examples the model
 * still gets wrong.  Such a row reaches the weights only through sums over the
 * batch, where it is lost in fp32 as well; its absolute error stays 2^-39 of the
 * tensor's maximum, only its error relative to its own size is not held at
 * 1e-5.  dlb_ctx_set_guard_strict(ctx, 1), called before the model's first
 * batch, (or DLB_GUARD_STRICT=1 in the environment) guards those rows too, at
 * the price of the fp32 kernel for every input-gradient product once the rows
 * have spread. */
dlb_status dlb_split_planes_2d(dlb_ctx *ctx, const float *x, float *planes, int rows, int cols);
dlb_status dlb_ctx_guard_counters(dlb_ctx *ctx, uint64_t *tensors_flagged, uint64_t *products_on_fallback);
dlb_status dlb_ctx_set_guard_strict(dlb_ctx *ctx, int strict);
/* Tensors whose planes were written a second time because the tensor had grown
 * more than eightfold since its previous split, beyond the scale predicted for
 * it (entry points that write planes in the producing kernel use that scale):
 * the check after the producer then splits the tensor again with the scale of
 * its own maximum, so that no product has to leave the tensor cores for it. */
dlb_status dlb_ctx_guard_resplits(dlb_ctx *ctx, uint64_t *tensors_resplit);

/* ------------------------------------------------------------------------ */
/* FC GEMMs. */

/* Z[b,o] = sum_i X[b,i] * W[o,i]  (+ bias[o] when bias != NULL).
 * ref: Model::Forward_Pass__FC__OpenMP (v1/learner/fwp_mp.cpp L:4419-4459) and
 * Forward_Pass__Bias__OpenMP (L:4396-4417). */
dlb_status dlb_fc_forward(dlb_ctx *ctx, const float *X, const float *X_lo, const float *W,
                          const float *W_lo, const float *bias, float *Z, int rows, int n_in,
                          int n_out);

/* dX[b,i] = sum_o delta[b,o] * W[o,i].
 * ref: Model::Backward_Pass__FC__OpenMP (v1/learner/bwp_mp.cpp L:968-1007). */
dlb_status dlb_fc_backward_input(dlb_ctx *ctx, const float *delta, const float *delta_lo,
                                 const float *W, const float *W_lo, float *dX, int rows,
                                 int n_in, int n_out);

/* dW[o,i] (+)= sum_b delta[b,o] * X[b,i];  dbias[o] (+)= sum_b delta[b,o] when
 * dbias != NULL.  accumulate != 0 adds to dW/dbias, else overwrites.
 * ref: Model::Update_Derivative_Weight__FC__OpenMP
 * (v1/learner/update_derivative_fwp_mp.cpp L:175-213) and ...__Bias (L:215-240).
 * Where n_out is not a multiple of 64 (and the product is large enough for the
 * tensor cores) the planes of delta are not used: the call makes planes of its
 * own for this product, one scale per unit o, from the fp32 tensor.  Inside a
 * model the weight gradient of a softmax output layer takes the same path
 * whatever its width, because the errors of its classes differ by many orders
 * of magnitude. */
dlb_status dlb_fc_weight_gradient(dlb_ctx *ctx, const float *delta, const float *delta_lo,
                                  const float *X, const float *X_lo, float *dW, float *dbias,
                                  int rows, int n_in, int n_out, int accumulate);

/* ------------------------------------------------------------------------ */
/* Batch renormalization. */

/* Per-unit statistics and corrections of one layer at one time step; every
 * pointer addresses n_units floats. */
typedef struct dlb_brn_unit_arrays {
  float *mean;          /* batch mean                                   */
  float *sigma;         /* batch standard deviation sqrt(E[x^2]-mu^2+eps) */
  float *mean_average;  /* running mean                                 */
  float *sigma_average; /* running standard deviation                   */
  float *r;             /* r correction                                 */
  float *d;             /* d correction                                 */
  const float *gamma;   /* scale (inside the parameter vector)          */
  const float *beta;    /* shift (inside the parameter vector)          */
} dlb_brn_unit_arrays;

/* sums[0..n) = sum_b Z[b,h], sums[n..2n) = sum_b Z[b,h]^2 over this rank's
 * rows, in double.  ref: the "Summation" loop of
 * Model::Forward_Pass__Batch_Renormalization__Training__OpenMP
 * (v1/learner/fwp_mp.cpp L:4647-4663). */
dlb_status dlb_brn_forward_sums(dlb_ctx *ctx, const float *Z, int rows, int n_units,
                                double *sums);

/* Same sums as dlb_brn_forward_sums for callers that must not allocate device
 * memory: code running between cudaStreamBeginCapture and EndCapture, inside a
 * host callback or a latency-critical loop where cudaMalloc would serialise
 * the device, or under a framework allocator that owns every byte of the GPU
 * and treats foreign allocations as a bug.  dlb_brn_forward_sums may grow the
 * context's scratch arena with cudaMalloc; this variant keeps its per-chunk
 * partial sums in an array that is part of the library image on every GPU that
 * loads it (DLB_NOALLOC_SCRATCH_DOUBLES doubles = 8 MiB, held until the process
 * exits) and calls no cudaMalloc, cudaFree or allocating routine.  It needs no
 * context: pass the stream to enqueue on (NULL = the default stream) with the
 * target device current.  Has no counterpart in the reference.
 *
 * Limits and rules:
 *  - the partial sums of one call must fit: row_chunks * 2 * n_units <=
 *    DLB_NOALLOC_SCRATCH_DOUBLES, where row_chunks <= ceil(4 * SM count /
 *    ceil(n_units / 128)) and <= ceil(rows / 64).  Larger requests return
 *    DLB_ERR_INVALID with a message naming both numbers; nothing is launched.
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress) and the SM count; make that first call outside any
 *    stream capture.
 *  - every call on a device shares the one array.  Nothing in it needs to
 *    start at zero (each call overwrites every slot it later reads), but two
 *    calls that overlap on the GPU (different streams) race on it: order them.
 *  - Z must be 16-byte aligned when n_units is a multiple of 4. */
#define DLB_NOALLOC_SCRATCH_DOUBLES (1u << 20)
dlb_status dlb_brn_forward_sums_noalloc(const float *Z, int rows, int n_units, double *sums,
                                        void *stream);

/* From (all-reduced) sums over global_rows rows: mean, sigma, running averages
 * (updated first), then r and d from the updated averages.
 * ref: the "Average" loop, fwp_mp.cpp L:4666-4718. */
dlb_status dlb_brn_forward_finalize(dlb_ctx *ctx, const double *sums, int global_rows,
                                    int n_units, float momentum, float epsilon, float r_max,
                                    float d_max, const dlb_brn_unit_arrays *u);

/* Dropout applied in place on the activation, as the reference does. */
typedef struct dlb_dropout_desc {
  int type;              /* DLB_DROPOUT_* */
  float value;           /* Bernoulli: keep probability; UOut: unused */
  const uint8_t *mask;   /* [n_units], one flag per unit shared by all rows */
  const float *noise;    /* UOut: [rows, n_units] draws of U(-p, p) */
} dlb_dropout_desc;

/* x_hat = (Z-mean)/sigma*r + d; y = gamma*x_hat + beta (u != NULL), else y = Z;
 * A = f(y); dropout in place.  A_lo (optional) receives the TF32 residual
 * plane of A for the next GEMM.
 * ref: the "Activation function" loop of the BRN forward (fwp_mp.cpp
 * L:4721-4738), Forward_Pass__FC_AF__OpenMP (L:4741-4770, AF_FIRE in
 * v1/ops/activations/functions.hpp L:124-219) and the dropout forwards
 * (fwp_mp.cpp L:4809-4868, L:4959-4985). */
dlb_status dlb_activation_forward(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                                  int af, const dlb_dropout_desc *dropout, float *A,
                                  float *A_lo, int rows, int n_units);

/* Row softmax.  ref: Forward_Pass__FC_AF__Softmax__OpenMP (fwp_mp.cpp L:4772-4807). */
dlb_status dlb_softmax_forward(dlb_ctx *ctx, const float *Z, float *Q, int rows, int n_units);

/* delta_af = dA * f'(y, A) written over dA, with y recomputed from Z as in
 * the forward pass.  With u != NULL also the four per-unit sums of the batch
 * renormalization backward over this rank's rows, in double:
 * sums[0..n) d_gamma, [n..2n) d_beta, [2n..3n) d_mean, [3n..4n) d_sigma.
 * ref: Backward_Pass__FC__DF__OpenMP (v1/learner/bwp_mp.cpp L:1150-1186),
 * Model::activation_fn_derivative (v1/learner/model.cpp L:2594-2650) and pass
 * 1 of Backward_Pass__Batch_Renormalization__OpenMP (bwp_mp.cpp L:1543-1578). */
dlb_status dlb_activation_backward(dlb_ctx *ctx, float *dA, const float *Z, const float *A,
                                   const dlb_brn_unit_arrays *u, int af, int rows, int n_units,
                                   double *sums);

/* dlb_fc_forward followed by dlb_activation_forward of a layer WITHOUT
 * normalization, as one call: Z = X W^T + bias, A = dropout(f(Z)) (+ A's plane
 * buffer).  ref: Forward_Pass__FC__OpenMP + Forward_Pass__Bias__OpenMP +
 * Forward_Pass__FC_AF__OpenMP and the dropout forwards (v1/learner/fwp_mp.cpp
 * L:4396-4459, L:4741-4770, L:4809-4985).  Where the product runs on the 2-CTA
 * tensor-core kernel (fp16 planes, at least 256 x 256 outputs, both operands'
 * plane buffers kept by the caller, A's buffer split once before), bias,
 * activation, dropout (Bernoulli flags per unit, inverted Bernoulli, UOut) and
 * the planes of A are formed in the product's epilogue, on the tile the drain
 * warps hold: A is never re-read.  Otherwise the two kernels run one after the
 * other; results are the same either way. */
dlb_status dlb_fc_forward_activation(dlb_ctx *ctx, const float *X, const float *X_lo, const float *W,
                                     const float *W_lo, const float *bias, float *Z, int af,
                                     const dlb_dropout_desc *dropout, float *A, float *A_lo, int rows,
                                     int n_in, int n_out);

/* dlb_fc_backward_input followed by dlb_activation_backward of the layer below
 * when that layer has NO normalization, as one call: dX = (delta W) * f'(Z_below,
 * A_below), the error of the layer below w.r.t. its sums (+ its plane buffer).
 * ref: Backward_Pass__FC__OpenMP + Backward_Pass__FC__DF__OpenMP
 * (v1/learner/bwp_mp.cpp L:968-1007, L:1150-1186).  Fused into the product's
 * epilogue under the conditions of dlb_fc_forward_activation. */
dlb_status dlb_fc_backward_input_derivative(dlb_ctx *ctx, const float *delta, const float *delta_lo,
                                            const float *W, const float *W_lo, const float *Z_below,
                                            const float *A_below, int af_below, float *dX, float *dX_lo,
                                            int rows, int n_in, int n_out);


/* delta = delta_af*gamma*r/sigma + d_sigma*(Z-mean)/(N*sigma) + d_mean/N over
 * delta (in place), N = global_rows; d_mean/d_sigma are sums[2n..4n) after the
 * all-reduce.  delta_lo optional.  ref: pass 3, bwp_mp.cpp L:1600-1626. */
dlb_status dlb_brn_backward_apply(dlb_ctx *ctx, float *delta, float *delta_lo, const float *Z,
                                  const dlb_brn_unit_arrays *u, const double *sums,
                                  int global_rows, int rows, int n_units);

/* d_gamma (+)= sums[0..n), d_beta (+)= sums[n..2n) as floats into the gradient
 * vector.  ref: the accumulation into ptr_array_derivatives_scales/shifts,
 * bwp_mp.cpp L:1559-1565. */
dlb_status dlb_brn_backward_param_grads(dlb_ctx *ctx, const double *sums, int n_units,
                                        float *d_gamma, float *d_beta, int accumulate);

/* ------------------------------------------------------------------------ */
/* Residual block (shortcut and block of equal width).
 * Forward: on rows with row_mask[b] != 0 every element of block[b,:] is
 * multiplied by noise[b,:] (draws of U(-1,1)), in place as the reference
 * perturbs the block's output buffer; out = x + block; out_lo optional.
 * row_mask == NULL: plain shortcut sum.
 * ref: Forward_Pass__Dropout__ShakeDrop__OpenMP (v1/learner/fwp_mp.cpp
 * L:4922-4957) and Forward_Pass__Zero_Padded_Identity__OpenMP (L:5058-5123). */
dlb_status dlb_residual_forward(dlb_ctx *ctx, const float *x, float *block,
                                const uint8_t *row_mask, const float *noise, float *out,
                                float *out_lo, int rows, int width);
/* Backward: delta = d * noise (draws of U(0,1)) on the rows perturbed forward,
 * d elsewhere; delta_lo optional.
 * ref: Backward_Pass__Dropout__ShakeDrop__OpenMP (v1/learner/bwp_mp.cpp L:933-966). */
dlb_status dlb_shakedrop_backward(dlb_ctx *ctx, const float *d, const uint8_t *row_mask,
                                  const float *noise, float *delta, float *delta_lo, int rows,
                                  int width);
/* The same pair where the block maps its input to another width.  The output is
 * as wide as the wider of x and block, W = max(width_x, width_block); the
 * narrower one enters from column pad = (|width_x - width_block| + 1) / 2 on
 * (v1/learner/compile.cpp L:337-352, Forward_Pass__Zero_Padded_Identity__OpenMP,
 * fwp_mp.cpp L:5058-5123).  Backward, each of the two reads its window of the
 * error d [rows, width_d]: columns first .. first + width
 * (Backward_Pass__Residual__OpenMP, bwp_mp.cpp L:1078-1140). */
dlb_status dlb_residual_forward_padded(dlb_ctx *ctx, const float *x, int width_x, float *block,
                                       int width_block, const uint8_t *row_mask,
                                       const float *noise, float *out, float *out_lo, int rows);
dlb_status dlb_shakedrop_backward_window(dlb_ctx *ctx, const float *d, int width_d, int first,
                                         const uint8_t *row_mask, const float *noise,
                                         float *delta, float *delta_lo, int rows, int width);

/* ------------------------------------------------------------------------ */
/* Recurrent (IndRNN) step.  Tensors are [seq_w, rows, n] row-major, the
 * reference's order (time step, example, unit: v1/learner/fwp_rec_mp.cpp
 * L:774-775).  With batch renormalization every time step has statistics of
 * its own: the six arrays of dlb_brn_unit_arrays then address seq_w * n floats
 * ([seq_w, n], v1/learner/allocate.cpp L:1348-1356), gamma and beta n floats.
 * Per-(t, unit) sums are laid out sums[(s * seq_w + t) * n + h]. */

/* [rows, seq_w * n] (one example per row, as the reference's callers hold
 * their data) -> [seq_w, rows, n]; out_lo optional.  Replaces the per-example
 * copy of Model::assign_inputs_rec_mp (v1/learner/assign_inputs.cpp L:199-225). */
dlb_status dlb_time_major(dlb_ctx *ctx, const float *x, float *out, float *out_lo, int rows,
                          int seq_w, int n);

/* s = 0: sum_b Z, s = 1: sum_b Z^2 for every (t, unit), in double.
 * ref: Forward_Pass__Batch_Renormalization__Training__OpenMP, reached once per
 * time step from Recurrent__Forward_Pass__FC__OpenMP (v1/learner/fwp_rec_mp.cpp
 * L:335-348; the sums loop is fwp_mp.cpp L:4647-4663). */
dlb_status dlb_brn_time_forward_sums(dlb_ctx *ctx, const float *Z, int seq_w, int rows, int n,
                                     double *sums);
/* dlb_brn_forward_finalize for all time steps at once. */
dlb_status dlb_brn_time_forward_finalize(dlb_ctx *ctx, const double *sums, int global_rows,
                                         int seq_w, int n, float momentum, float epsilon,
                                         float r_max, float d_max, const dlb_brn_unit_arrays *u);

/* y_t = batch-renormalised Z_t (u != NULL) or Z_t; pre_t = y_t + recurrent *
 * A_{t-1} (t = 0, or recurrent == NULL: pre_t = y_t); A_t = f(pre_t).
 * ref: Forward_Pass__FC_Ind_RNN__OpenMP (v1/learner/fwp_rec_mp.cpp L:762-800)
 * and the activation that follows it (L:335-348). */
dlb_status dlb_indrnn_forward(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                              const float *recurrent, int af, float *A, float *A_lo, int seq_w,
                              int rows, int n);
/* The same walk with Bernoulli dropout: the output of time step t is masked by
 * mask[t * n + unit] (kept units times keep_scale: 1, or 1 / p for the inverted
 * form) before it is stored, so the recurrence of step t + 1 reads the masked
 * value (fwp_mp.cpp L:1228-1262, L:4842-4868).  mask == NULL scales every unit
 * by keep_scale, the inference form (fwp_rec_mp.cpp L:299-312). */
dlb_status dlb_indrnn_forward_dropout(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                                      const float *recurrent, int af, const uint8_t *mask,
                                      float keep_scale, float *A, float *A_lo, int seq_w, int rows,
                                      int n);

/* The same walk with UOut: the output of time step t becomes h + h * noise[t,
 * row, unit] (draws of U(-beta, beta), [seq_w, rows, n]) before it is stored and
 * before the recurrence of step t + 1 reads it (fwp_mp.cpp L:1252-1257,
 * L:4959-4985). */
dlb_status dlb_indrnn_forward_uout(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                                   const float *recurrent, int af, const float *noise, float *A, float *A_lo,
                                   int seq_w, int rows, int n);

/* E holds dA on entry and dAF on return, t from seq_w-1 down to 0:
 *   f'_t = f'(pre_t, A_t), dAF_t = dA_t f'_t + recurrent f'_t dAF_{t+1}.
 * ref: Backward_Pass__FC__DF_Ind_RNN__OpenMP (v1/learner/bwp_mp.cpp L:1188-1263). */
dlb_status dlb_indrnn_backward_walk(dlb_ctx *ctx, float *E, const float *Z, const float *A,
                                    const dlb_brn_unit_arrays *u, const float *recurrent, int af,
                                    int seq_w, int rows, int n);

/* Per-(t, unit) sums over dAF.  With u != NULL, s = 0..3 are d_gamma, d_beta,
 * d_mean, d_sigma of the batch renormalization backward (bwp_mp.cpp
 * L:1543-1578); with recurrent != 0 the last s is sum_b A_{t-1} dAF_t (0 at
 * t = 0), the recurrent-weight gradient of that time step
 * (Update_Derivative_Weight__FC_Ind_RNN__OpenMP,
 * v1/learner/update_derivative_rec_mp.cpp L:460-487). */
dlb_status dlb_indrnn_backward_sums(dlb_ctx *ctx, const float *E, const float *Z, const float *A,
                                    const dlb_brn_unit_arrays *u, int recurrent, int seq_w,
                                    int rows, int n, double *sums);
/* out[h] += sum_t sums[t * n + h], t from seq_w-1 down to 0. */
dlb_status dlb_time_fold(dlb_ctx *ctx, const double *sums, int seq_w, int n, float *out);

/* dlb_brn_backward_apply for all time steps at once; sums as written by
 * dlb_indrnn_backward_sums (s = 2, 3 already summed over the ranks). */
dlb_status dlb_brn_time_backward_apply(dlb_ctx *ctx, float *delta, float *delta_lo, const float *Z,
                                       const dlb_brn_unit_arrays *u, const double *sums,
                                       int global_rows, int seq_w, int rows, int n);

/* LSTM layer, the parts that are not matrix products (lstm.cu).  Gates' sums and
 * gates' errors of a time step are rows of G = C + 3 B values {z of every cell | i
 * | f | o of every block}, C = blocks * cells; peep = {p_i | p_f | p_o}, C each.
 * forward_step: one time step from the sums g_in = W x_t and g_rec = R h_{t-1}
 * (NULL with c_prev at t = 0).  backward_step: the gates' errors d of one time
 * step from dH (error of the outputs, recurrent part included), what follows it
 * (gf_next, dC_next, d_next: NULL at the last step) and c_prev (NULL at t = 0).
 * peephole_gradient: out [3, C] from all time steps' errors d [seq_w, rows, G]
 * and states c [seq_w, rows, C].  gather_rows / scatter_add_rows move rows of
 * `width` floats between a packed matrix and offsets in a flat vector. */
dlb_status dlb_gather_rows(dlb_ctx *ctx, const float *src, const unsigned long long *offsets, float *dst,
                           size_t rows, int width);
dlb_status dlb_scatter_add_rows(dlb_ctx *ctx, const float *src, const unsigned long long *offsets, float *dst,
                                size_t rows, int width);
dlb_status dlb_lstm_forward_step(dlb_ctx *ctx, const float *g_in, const float *g_rec, const float *bias,
                                 const float *peep, const float *c_prev, float *z, float *c, float *ca, float *h,
                                 float *gi, float *gf, float *go, int rows, int blocks, int cells);
dlb_status dlb_lstm_backward_step(dlb_ctx *ctx, const float *dH, const float *z, const float *ca, const float *gi,
                                  const float *gf, const float *go, const float *c_prev, const float *gf_next,
                                  const float *dC_next, const float *d_next, const float *peep, float *dC, float *d,
                                  int rows, int blocks, int cells);
dlb_status dlb_lstm_peephole_gradient(dlb_ctx *ctx, const float *d, const float *c, float *out, int seq_w, int rows,
                                      int blocks, int cells);

/* recurrent[h] = clip(recurrent[h], lo, hi).
 * ref: Model::Update_Weight_Regularization__Constraint_Recurrent_Weight
 * (v1/ops/constraints/constraint.cpp L:245-289). */
dlb_status dlb_indrnn_clamp(dlb_ctx *ctx, float *recurrent, int n, float lo, float hi);

/* ------------------------------------------------------------------------ */
/* Output error and loss.
 * MSE: delta = f'(pre, q) * 2 (q - y) / (global_rows * n_out); loss += (q-y)^2.
 * Cross-entropy on a softmax layer: delta_j = sum_k (q_j [j==k] - q_k q_j) L'_k,
 * L'_k = (y_k == 1 ? -1/clip(q_k, 1e-7, 1-1e-7) : 0) / global_rows;
 * loss += (y==1 ? -log(clip(q)) : 0).  *loss_sum (device, double) accumulates.
 * ref: Model::compute_error_fwp_mp (v1/learner/compute_error_mp.cpp L:28-141),
 * loss_fn / loss_fn_derivative (v1/learner/compute_loss.cpp L:55-138). */
dlb_status dlb_loss_delta(dlb_ctx *ctx, int loss, int af, const float *pre, const float *q,
                          const float *y, float *delta, float *delta_lo, int rows, int n_out,
                          int global_rows, double *loss_sum);

/* Evaluation: loss_sum += the loss of every output against its target (as
 * dlb_loss_delta accumulates it) and accu_sum += the accuracy count: DISTANCE:
 * elements with |q - y| <= accu_var; CROSS_ENTROPY: rows whose largest output
 * (the last of equal maxima) sits where the target is 1.  No error is formed.
 * ref: compute_loss_fwp_mp (v1/learner/compute_loss_mp.cpp L:28-113). */
dlb_status dlb_loss_eval(dlb_ctx *ctx, int loss, int accu_fn, float accu_var, const float *q,
                         const float *y, int rows, int n_out, double *loss_sum, double *accu_sum);

/* ------------------------------------------------------------------------ */
/* Optimizer: one pass over flat arrays of n elements; gradient zeroed after
 * use as the reference does. */
typedef struct dlb_optimizer_scalars {
  float lr_t;        /* lr * sqrt(1-beta2^t)/(1-beta1^t) (or lr without bias correction) */
  float beta1;
  float beta2;       /* NosAdam: beta2 at time t                          */
  float epsilon;
  float lower_bound; /* AdaBound / AMSBound                               */
  float upper_bound;
  float weight_decay;/* 0: off; else p -= ... + mask*wd*p                 */
} dlb_optimizer_scalars;

/* ref: Model::Update_Parameters__{Adam,AMSGrad,AdaBound,AMSBound,NosAdam}__OpenMP
 * (v1/optimizers/adam.cpp L:98-165, amsgrad.cpp L:34-109, adabound.cpp
 * L:38-112, amsbound.cpp L:38-126, nosadam.cpp L:33-102).  AdaMax has no
 * implementation in the reference (v1/learner/model.cpp L:4765-4767); the
 * rule here is Kingma & Ba section 7 with second = the infinity norm u.
 * DLB_OPT_GD is Model::Update_Parameter__Gradient_Descent
 * (v1/optimizers/gradient_descent.cpp L:24-130, gradient_descent_momentum.cpp
 * L:66-107, nesterov_accelerated_gradient.cpp L:66-109): lr_t = learning rate,
 * beta1 = momentum (0: plain descent, `first` unused), beta2 != 0 = the
 * Nesterov form; `first` holds the previous delta, `second` is unused. */
dlb_status dlb_optimizer_step(dlb_ctx *ctx, int rule, const dlb_optimizer_scalars *s, float *p,
                              float *g, float *first, float *second, float *second_hat,
                              const float *wd_mask, size_t n);

/* Gradient clipping by the Euclidean norm of g[0..n): g *= max_norm / |g| when
 * |g| >= max_norm.  ref: euclidean_norm_mp (v1/ops/constraints/euclidean.cpp
 * L:48-71) as Model::Clip_Gradient__OpenMP calls it between the merge and the
 * optimizer (v1/learner/model.cpp L:4742-4743).  The sum of squares is formed
 * in fp64 (the reference adds floats in thread order). */
dlb_status dlb_clip_gradient(dlb_ctx *ctx, float *g, size_t n, float max_norm);

/* Host-side scalars exactly as the reference derives them from its float time
 * step (increments *time_step first).  hyper = {lr, beta1, beta2, epsilon,
 * gamma(NosAdam), final_lr, bound_gamma, bias_correction(0/1)};
 * *nos_previous is NosAdam's running B_{t-1}.  For DLB_OPT_GD hyper =
 * {learning_rate, learning_momentum, use_nesterov(0/1)}. */
dlb_status dlb_optimizer_prepare(int rule, const float *hyper, float *time_step,
                                 float *nos_previous, dlb_optimizer_scalars *out);

/* ------------------------------------------------------------------------ */
/* Data-parallel exchange (NCCL over NVLink): sums over all ranks, in place,
 * on the context's stream.  With no communicator bound they are no-ops. */
dlb_status dlb_comm_unique_id(char out_id[128]);
dlb_status dlb_comm_init(dlb_ctx *ctx, const char id[128], int rank, int world);
int dlb_comm_world(dlb_ctx *ctx);
int dlb_comm_rank(dlb_ctx *ctx);
dlb_status dlb_allreduce_f32(dlb_ctx *ctx, float *buf, size_t n);
dlb_status dlb_allreduce_f64(dlb_ctx *ctx, double *buf, size_t n);
/* Same sum, enqueued on the context's second (communication) stream behind
 * everything already on the main stream, so that it overlaps with the kernels
 * the caller enqueues next (the gradient of one layer crosses NVLink while the
 * weight-gradient GEMM of the next layer runs).  dlb_comm_join makes the main
 * stream wait for all such transfers. */
dlb_status dlb_allreduce_f32_overlapped(dlb_ctx *ctx, float *buf, size_t n);
dlb_status dlb_comm_join(dlb_ctx *ctx);
/* dlb_allreduce_f64 of up to 32768 doubles (the batch-renormalization sums of
 * a layer: Forward_Pass__Batch_Renormalization__Training__OpenMP,
 * fwp_mp.cpp L:4647-4663, and the backward sums of bwp_mp.cpp L:1520-1621)
 * does not go through NCCL when the ranks are processes of one host on GPUs of
 * their own: dlb_comm_init maps a buffer of every rank into every rank (CUDA
 * IPC) and one kernel per rank stores its vector, every 8-byte word tagged
 * with the exchange's sequence number, into all of them over NVLink, waits
 * (bounded; DLB_ERR_TIMEOUT in the device status after 20 s) for the other
 * ranks' words and adds the vectors in rank order, so that all ranks hold the
 * same bits.  1 if the context uses it
 * (DLB_PEER_EXCHANGE=0 in the environment of any rank turns it off for all). */
int dlb_comm_peer_exchange(dlb_ctx *ctx);
/* The same protocol with `world` (<= 8) emulated ranks as the rows of one
 * cooperative grid on this device, for checking it where there is one GPU.
 * in/out: host arrays [world][n], n <= 32768; `rounds` exchanges run back to
 * back on the same buffers, round k on the vectors times k + 1, and `out` is
 * what each rank holds after the last.  absent >= 0 names a rank that never
 * delivers: the others give up after wait_ms and the call returns
 * DLB_ERR_TIMEOUT, the device status is cleared and the context stays usable. */
dlb_status dlb_peer_exchange_emulated(dlb_ctx *ctx, int world, size_t n, int rounds,
                                      const double *in, double *out, int absent,
                                      unsigned wait_ms);

/* ------------------------------------------------------------------------ */
/* Model: the reference's v1::Model construction and step entry points
 * (v1/learner/model.hpp L:752-3384) over the kernels above.  Same setter
 * names, argument meaning and call order; errors are status codes where the
 * reference returns false and logs. */
typedef struct dlb_model dlb_model;

dlb_status dlb_model_create(dlb_model **out, dlb_ctx *ctx);
dlb_status dlb_model_destroy(dlb_model *m);
/* ref: Model::compile (model.hpp L:2528). */
dlb_status dlb_model_compile(dlb_model *m, size_t n_layers, size_t seq_w, int model_type,
                             const int *layer_types, const size_t *layer_units);
/* compile() with Layer_Parameters::unit_parameters[1] of every layer
 * (layer_units2, may be NULL): the cells per memory block of an LSTM layer,
 * whose layer_units entry is its number of blocks (v1/learner/compile.cpp
 * L:98-118).  An LSTM layer (DLB_LAYER_LSTM) is unidirectional with peephole
 * connections, tanh on cell input and state, sigmoid gates
 * (v1/learner/fwp_rec_mp.cpp L:802-1526, bwp_rec_mp.cpp L:1006-1582,
 * update_derivative_rec_mp.cpp L:489-774), its parameters laid out block by
 * block and its biases indexed as the reference does
 * (connections_prepare.cpp L:83-262).  Not supported on it: normalization,
 * dropout, zoneout, the bidirectional form; saving a model with LSTM layers. */
dlb_status dlb_model_compile2(dlb_model *m, size_t n_layers, size_t seq_w, int model_type,
                              const int *layer_types, const size_t *layer_units, const size_t *layer_units2);
dlb_status dlb_model_set_layer_activation_function(dlb_model *m, size_t layer, int af);
dlb_status dlb_model_set_layer_normalization(dlb_model *m, size_t layer, int norm);
dlb_status dlb_model_set_dropout(dlb_model *m, size_t layer, int type, float value0,
                                 int scale_weights);
dlb_status dlb_model_set_normalization_momentum_average(dlb_model *m, float v);
dlb_status dlb_model_set_normalization_epsilon(dlb_model *m, float v);
dlb_status dlb_model_set_brn_r_correction_maximum(dlb_model *m, float v);
dlb_status dlb_model_set_brn_d_correction_maximum(dlb_model *m, float v);
dlb_status dlb_model_set_loss_fn(dlb_model *m, int loss);
dlb_status dlb_model_set_optimizer(dlb_model *m, int optimizer);
/* Public hyper-parameter fields of the reference's Model, by field name. */
dlb_status dlb_model_set_hparam(dlb_model *m, const char *name, double value);
double dlb_model_get_hparam(dlb_model *m, const char *name);
/* Decoupled weight decay on the weights (not on biases, scales, shifts), with
 * the reference's normalisation by sqrt(batch / (training_size * epoch)).
 * ref: Model::set_weight_decay (v1/ops/regularizers/weight_decay.cpp L:26-60),
 * Model::normalized_wd (v1/learner/train.cpp L:278-283). */
dlb_status dlb_model_set_weight_decay(dlb_model *m, float value);
/* ref: Model::set_l2 (v1/ops/regularizers/l2.cpp L:31-66).  Kept and written to
 * the hyperparameter file; like the reference's, the value never reaches the
 * gradient (its update calls the L2 routine over an empty index range:
 * v1/learner/model.cpp L:4717-4719 against l2.cpp L:92-104). */
dlb_status dlb_model_set_l2(dlb_model *m, float value);
dlb_status dlb_model_set_max_batch_size(dlb_model *m, size_t rows);
dlb_status dlb_model_set_seq_w(dlb_model *m, size_t time_delays);
dlb_status dlb_model_seed_weights(dlb_model *m, unsigned seed);
dlb_status dlb_model_initialize_weights_with_glorot_uniform(dlb_model *m);
size_t dlb_model_get_size(dlb_model *m, const char *name);
dlb_status dlb_model_layer_info(dlb_model *m, size_t layer, size_t out[10]);
/* name: parameters, derivatives, first_moment, second_moment,
 * second_moment_hat.  Host <-> device copies of the flat vectors
 * (the reference's Copy__Parameters__Device_To_Host, model.cpp L:2300-2351). */
dlb_status dlb_model_get_array(dlb_model *m, const char *name, float *host_out, size_t n);
dlb_status dlb_model_set_array(dlb_model *m, const char *name, const float *host_in, size_t n);
dlb_status dlb_model_get_layer_norm(dlb_model *m, size_t layer, const char *name, float *host_out,
                                    size_t n);
dlb_status dlb_model_set_layer_norm(dlb_model *m, size_t layer, const char *name,
                                    const float *host_in, size_t n);
dlb_status dlb_model_set_dropout_mask(dlb_model *m, size_t layer, const uint8_t *host_mask,
                                      size_t n);
/* This step's UOut draws for a layer whose dropout is DLB_DROPOUT_UOUT:
 * host_noise[rows, units] of U(-beta, beta); the forward pass computes
 * A += A * noise.  The reference draws them on the host inside the forward
 * pass (Forward_Pass__Dropout__Uout__OpenMP, v1/learner/fwp_mp.cpp
 * L:4959-4985); here they are an input, like the dropout masks. */
dlb_status dlb_model_set_uout_noise(dlb_model *m, size_t layer, const float *host_noise, size_t rows);
/* ShakeDrop draws of one training step for a RESIDUAL layer: row flags [rows]
 * and the forward U(-1,1) / backward U(0,1) draws [rows, width of the block's
 * last layer] (host arrays;
 * only flagged rows are read).  The reference draws them from clock-seeded
 * generators inside the step (fwp_mp.cpp L:4942-4955, bwp_mp.cpp L:959-963);
 * here they are inputs so that a run can be reproduced. */
dlb_status dlb_model_set_shakedrop_noise(dlb_model *m, size_t layer, const uint8_t *host_row_mask,
                                         const float *host_forward, const float *host_backward,
                                         size_t rows);
/* Data-parallel: rows given to forward_pass are this rank's shard of a batch
 * of global_rows rows (default: equal to the call's rows). */
dlb_status dlb_model_set_global_batch(dlb_model *m, size_t global_rows);
/* Examples in the training set: what dlb_model_train_step, _device and _staged
 * pass as training_size to dlb_model_update_weights (the normalised weight decay
 * is weight_decay * sqrt(batch / (training_size * epoch)), Model::normalized_wd,
 * v1/learner/train.cpp L:278-283).  0 (default): the batch is the whole set. */
dlb_status dlb_model_set_training_size(dlb_model *m, size_t training_size);

/* Step entry points; X/Y are HOST arrays of row pointers exactly as the
 * reference takes them (model.hpp L:2980, L:1054), each row seq_w*n values. */
dlb_status dlb_model_forward_pass(dlb_model *m, size_t rows, const float *const *Xm);
dlb_status dlb_model_compute_error(dlb_model *m, size_t rows, const float *const *Ym);
dlb_status dlb_model_backward_pass(dlb_model *m, size_t rows);
dlb_status dlb_model_update_derivatives(dlb_model *m, size_t rows);
/* Evaluation, as Driver::evalt (drivers/driver.cpp L:60-105): set the
 * propagation state to INFERENCE, run forward passes (normalization by the
 * running averages, fwp_mp.cpp L:4461-4491, every time step by its own in a
 * time-stepped model; plain Bernoulli dropout scales by its keep probability,
 * L:4870-4892; the block output of a ShakeDrop layer by 1 - p, L:3876-3897),
 * and after each one dlb_model_compute_loss
 * (Model::compute_loss, v1/learner/compute_loss.cpp L:140-161) accumulates the
 * loss and the accuracy counter without forming an error.  dlb_model_get_loss
 * and dlb_model_get_accuracy (percent, Model::get_accu) read them. */
dlb_status dlb_model_set_propagation(dlb_model *m, int state);
dlb_status dlb_model_set_accu_fn(dlb_model *m, int fn);
dlb_status dlb_model_set_accu_var(dlb_model *m, float v);
dlb_status dlb_model_compute_loss(dlb_model *m, size_t rows, const float *const *Ym);
dlb_status dlb_model_compute_loss_device(dlb_model *m, size_t rows, const float *Y_dev);
dlb_status dlb_model_get_accuracy(dlb_model *m, double *accuracy);
/* on = 1: dlb_model_compute_error keeps the accuracy counter as well, as
 * Model::compute_error does in the reference (compute_error_fwp_mp /
 * compute_error_rec_mp, v1/learner/compute_error_mp.cpp L:60-112, L:178-231):
 * one more pass over the outputs and targets per step; dlb_model_get_accuracy
 * then reads the accuracy of the training pass since dlb_model_reset_loss.
 * Default 0: training steps leave the counter alone. */
dlb_status dlb_model_set_training_accuracy(dlb_model *m, int on);
/* Across GPUs this is the gradient all-reduce (the reference's thread merge,
 * v1/learner/merge.cpp L:76-100). */
dlb_status dlb_model_merge_derivatives(dlb_model *m);
dlb_status dlb_model_update_weights(dlb_model *m, size_t rows, size_t training_size);
dlb_status dlb_model_get_loss(dlb_model *m, double *loss);
dlb_status dlb_model_reset_loss(dlb_model *m);
/* Same step with inputs already on the device, contiguous [rows, seq_w*n]. */
dlb_status dlb_model_forward_pass_device(dlb_model *m, size_t rows, const float *X_dev);
dlb_status dlb_model_compute_error_device(dlb_model *m, size_t rows, const float *Y_dev);
/* forward, error, backward, gradients, merge, update in one call.  X/Y are
 * contiguous host arrays [rows, seq_w*n]; copied through pinned staging. */
dlb_status dlb_model_train_step(dlb_model *m, size_t rows, const float *X_host,
                                const float *Y_host, double *loss);
dlb_status dlb_model_train_step_device(dlb_model *m, size_t rows, const float *X_dev,
                                       const float *Y_dev);
/* Noise drawn on the device instead of handed over by the host: a counter-based
 * generator (Philox4x32-10, Salmon et al., SC'11) in which element i of a draw
 * is a function of (seed, stream, step, first + i) alone.  dlb_noise_uniform
 * writes lo + (hi - lo) u with u = 24 random bits / 2^24; dlb_noise_bernoulli
 * writes 1 where u < p.  dlb_model_draw_noise fills, for the next step of
 * `rows` rows, every layer's Bernoulli mask (one flag per unit, kept with the
 * layer's probability), UOut draws U(-beta, beta) and ShakeDrop flags and
 * factors; rows are numbered from first_row, the rank's first row in the whole
 * batch, so that the draws do not depend on the sharding.  The reference draws
 * the same distributions from per-thread std::mt19937 streams during the step
 * (Model::Dropout_Bernoulli; fwp_mp.cpp L:4959-4985, L:4922-4957); its streams
 * depend on the thread count, the host-array setters reproduce them. */
dlb_status dlb_noise_uniform(dlb_ctx *ctx, float *out, size_t n, float lo, float hi, uint64_t seed,
                             uint32_t stream, uint32_t step, uint64_t first);
dlb_status dlb_noise_bernoulli(dlb_ctx *ctx, uint8_t *out, size_t n, float p, uint64_t seed,
                               uint32_t stream, uint32_t step, uint64_t first);
dlb_status dlb_model_draw_noise(dlb_model *m, size_t rows, uint64_t seed, uint32_t step,
                                size_t first_row);
/* The reference's on-disk format.  dlb_model_save_params writes what
 * Model::save_params writes (dimensions, layers, normalization state and every
 * weight as text; v1/learner/save.cpp L:188-520) and dlb_model_save_spec_params
 * what Model::save_spec_params writes (hyperparameters; L:34-186; values of
 * options outside the supported path as the reference's defaults), so that the
 * reference's Model::load reads a model trained here.  dlb_model_load reads the
 * pair into a model that has not been compiled yet (Model::load,
 * v1/learner/load.cpp L:1243-); a file that uses a layer type, regularizer or
 * option outside the supported path is refused.  Optimizer moments are not
 * part of the reference's format and are not written. */
dlb_status dlb_model_save_params(dlb_model *m, const char *path);
dlb_status dlb_model_save_spec_params(dlb_model *m, const char *path);
dlb_status dlb_model_load(dlb_model *m, const char *path_params, const char *path_spec);
/* Checkpoint directories with rotation, in the reference's layout
 * (DL::Checkpointer, nn/checkpointer.cpp L:41-221): <dir>/ckpt-<step>/model.net
 * and model.nn (the two files above), <dir>/checkpoint naming the newest, the
 * newest max_to_keep directories kept.  The library adds <dir>/ckpt-<step>/
 * model.opt, the optimizer's moments and time step, which the reference's format
 * lacks and its loader ignores; dlb_checkpointer_load restores them when present.
 * dlb_checkpointer_step is CheckpointerInterval::operator() (L:230-250): saves
 * (as step_train) when forced, or when g has reached the next due step and
 * is_top is set, then moves the due step to g + interval.
 * dlb_checkpointer_load wants a model that has not been compiled; *found = 0 when
 * the directory holds no checkpoint. */
typedef struct dlb_checkpointer dlb_checkpointer;
dlb_status dlb_checkpointer_create(dlb_checkpointer **out, dlb_model *model, const char *ckpt_dir,
                                   int max_to_keep, int interval);
dlb_status dlb_checkpointer_destroy(dlb_checkpointer *c);
dlb_status dlb_checkpointer_save(dlb_checkpointer *c, int step_train);
dlb_status dlb_checkpointer_step(dlb_checkpointer *c, int g, int step_train, int is_top, int force, int *saved);
dlb_status dlb_checkpointer_load(dlb_checkpointer *c, int *found);
/* The mini-batch loop around the step: DL::v1::MiniBatch
 * (v1/data/dataset/minibatch.cpp).  Xm / Ym are the data set's arrays of row
 * pointers (n_examples rows of seq_w * n_in and seq_w * n_out floats; they must
 * stay valid while the object lives).  Batches as Set__Desired_Data_Per_Batch
 * makes them (L:118-190): floor(n_examples / desired_per_batch) of them, at most
 * max_batches when that is not 0, the last one larger by the remainder as the
 * reference takes it, (n / desired - batches) * desired in double and truncated
 * (330 rows in batches of 100 give 100, 100 and 129: the product is 29.99...);
 * fewer than two batches are refused as in the reference.  Shuffle (L:42-58) is the
 * reference's Fisher-Yates pass with std::mt19937 and
 * std::uniform_int_distribution; the reference seeds it from the clock, here
 * the seed is an argument.  dlb_minibatch_train is MiniBatch::train_mp (L:286-323):
 * shuffle if asked, then per batch one training step with
 * update_weights(rows of the batch, rows of the data set) and its loss read;
 * epoch_time_step + 1; *loss = mean of the batch losses.  Batch k + 1 is
 * gathered into page-locked memory and copied to the device while batch k
 * trains (dlb_model_stage_batch).  train_mp also adds up the accuracy of every
 * batch (for the accuracy functions supported here DatasetV1::compute_accuracy
 * returns the counter the training pass kept,
 * v1/data/dataset/dataset_v1.cpp L:4540-4640): dlb_minibatch_get_accuracy
 * returns its mean over the batches of the last pass, in percent, the value
 * train_mp hands to Model::set_accu(ENV::TRAIN, ...). */
typedef struct dlb_minibatch dlb_minibatch;
dlb_status dlb_minibatch_create(dlb_minibatch **out, dlb_model *model, const float *const *Xm,
                                const float *const *Ym, size_t n_examples, int use_shuffle,
                                size_t desired_per_batch, size_t max_batches, unsigned seed);
dlb_status dlb_minibatch_destroy(dlb_minibatch *mb);
size_t dlb_minibatch_get_n_batch(const dlb_minibatch *mb);
size_t dlb_minibatch_examples_per_batch(const dlb_minibatch *mb);
size_t dlb_minibatch_examples_last_batch(const dlb_minibatch *mb);
dlb_status dlb_minibatch_set_shuffle(dlb_minibatch *mb, int use_shuffle);
dlb_status dlb_minibatch_shuffle(dlb_minibatch *mb);
/* The current order of the rows (MiniBatch::ptr_array_stochastic_index), n = n_examples. */
dlb_status dlb_minibatch_get_order(const dlb_minibatch *mb, size_t *out, size_t n);
dlb_status dlb_minibatch_train(dlb_minibatch *mb, double *loss);
double dlb_minibatch_get_accuracy(const dlb_minibatch *mb);

/* Model::set_clip_gradient, both overloads (v1/ops/constraints/clip_gradient.cpp
 * L:30-73): whether update_weights clips, and the norm; the norm also sets the
 * default bound of IndRNN recurrent weights, clip(value, 2, 10)^(1/seq_w)
 * (v1/ops/constraints/constraint.cpp L:64-95). */
dlb_status dlb_model_set_clip_gradient(dlb_model *m, int use, float value);
/* Model::Set__Regularization__Constraint_Recurrent_Weight(index, lower, upper)
 * and its __Default form (v1/ops/constraints/constraint.cpp L:97-243): the bounds
 * the recurrent weights of one IndRNN layer are clamped to after every update
 * (L:245-289).  Hidden layers with recurrent weights only, lower <= upper; 0 / 0
 * takes the clamp off.  Without a call the default applies and follows
 * set_clip_gradient, as in the reference; bounds equal to the default (within
 * 1e-8) count as the default.  The bounds are written to and read from the
 * parameter file like the reference's. */
dlb_status dlb_model_set_constraint_recurrent_weight(dlb_model *m, size_t layer, float lower, float upper);
dlb_status dlb_model_set_constraint_recurrent_weight_default(dlb_model *m, size_t layer);
dlb_status dlb_model_get_constraint_recurrent_weight(dlb_model *m, size_t layer, float *lower, float *upper);
/* The same step with the input copy taken off the critical path.  stage_batch
 * starts the host-to-device copy of one batch (contiguous [rows, seq_w*n]
 * arrays, page-locked for the copy to be asynchronous; they must stay
 * untouched until the step that uses them has been called) on a stream of its
 * own and returns; up to two batches may be staged.  train_step_staged runs
 * the step on the oldest staged batch.  Staging batch i+1 before stepping on
 * batch i hides the copy under the kernels.  This is the mini-batch loop of
 * MiniBatch::train_mp (v1/data/dataset/minibatch.cpp L:286-323): train on the
 * batch, read its loss, update the weights, move to the next batch. */
dlb_status dlb_model_stage_batch(dlb_model *m, size_t rows, const float *X_host,
                                 const float *Y_host);
dlb_status dlb_model_train_step_staged(dlb_model *m, double *loss);
/* steps = 1: dlb_model_train_step_staged returns the loss of the step before the
 * one it has just enqueued (NaN on the first call), so that the host never
 * waits for the device inside the loop and runs one step ahead of it;
 * dlb_model_get_loss after the loop reads the last step's.  steps = 0
 * (default): the loss of the step itself, for which the host waits after it
 * has enqueued the update. */
dlb_status dlb_model_set_loss_lag(dlb_model *m, int steps);
/* Several ranks, one-call steps (dlb_model_train_step*) of a plain stack of
 * fully connected layers.  on = 1 (default): where the rows of every weight
 * matrix divide evenly among the ranks and the gradient is not clipped by its
 * norm, the merge of Model::merge_mp_derivatives (v1/learner/merge.cpp L:76-100)
 * and the update of Model::update_weights_mp (v1/learner/model.cpp L:4711-4796)
 * are done owner by owner: the gradient of a matrix is reduce-scattered by rows,
 * each rank updates weights and moments of its rows, the updated rows are
 * gathered; every rank ends the step with the same weights as with the
 * replicated update, element for element the same arithmetic.  The moments of
 * the matrices are then current only on their owners until they are read
 * (dlb_model_get_array of a moment vector, the moments file of a checkpoint, a
 * later replicated update): those calls gather them and are collective, every
 * rank makes them at the same point.  on = 0: all-reduce and the same update on
 * every rank.  The environment variable DLB_SHARDED_UPDATE=0 has the same
 * effect for every model of the process. */
dlb_status dlb_model_set_sharded_update(dlb_model *m, int on);
dlb_status dlb_model_get_layer_outputs(dlb_model *m, size_t layer, size_t rows, float *host_out);
dlb_status dlb_model_get_layer_errors(dlb_model *m, size_t layer, size_t rows, int which,
                                      float *host_out);

#ifdef __cplusplus
}
#endif
#endif /* DLB200_H_ */
