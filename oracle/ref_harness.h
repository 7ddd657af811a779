/* Test infrastructure, not product code.
 *
 * C entry points of oracle/_ref/libdlref.so: a thin driver around the
 * reference library's own DL::v1::Model, so that a Python test (ctypes) can
 * build a model with the reference's setters, inject seeded inputs, weights
 * and dropout masks, run the reference's OpenMP training step and read back
 * every tensor that the CUDA path is compared with.
 *
 * Integer codes for layer / activation / normalisation / dropout / optimizer /
 * loss are the numeric values of the reference's enums
 * (lib/deep-learning/v1/data/enum/{layer,activation,layer_norm,layer_dropout,
 * optimizer,loss_fn,model}.hpp).  All functions returning int give 0 on
 * success and -1 on failure.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *ref_model;

ref_model ref_model_create(void);
void ref_model_destroy(ref_model m);

int ref_compile(ref_model m, size_t n_layers, size_t seq_w, int model_type,
                const int *layer_types, const size_t *layer_units,
                size_t allowable_memory);
int ref_compile2(ref_model m, size_t n_layers, size_t seq_w, int model_type, const int *layer_types,
                 const size_t *layer_units, const size_t *layer_units2, size_t allowable_memory);
int ref_set_layer_activation_function(ref_model m, size_t layer, int af);
int ref_set_layer_normalization(ref_model m, size_t layer, int norm);
int ref_set_dropout(ref_model m, size_t layer, int type, float value0,
                    int scale_weights);
int ref_set_normalization_momentum_average(ref_model m, float v);
int ref_set_normalization_epsilon(ref_model m, float v);
int ref_set_brn_r_correction_maximum(ref_model m, float v);
int ref_set_brn_d_correction_maximum(ref_model m, float v);
int ref_set_loss_fn(ref_model m, int loss);
int ref_set_optimizer(ref_model m, int optimizer);
/* name: adam_learning_rate, adam_beta1, adam_beta2, adam_epsilon, adam_gamma,
 * learning_rate_final, learning_gamma, use_adam_bias_correction,
 * weight_decay, pct_threads. */
int ref_set_hparam(ref_model m, const char *name, double value);
double ref_get_hparam(ref_model m, const char *name);
int ref_set_max_batch_size(ref_model m, size_t b);
int ref_set_mp(ref_model m, int use_mp);
int ref_set_weight_decay(ref_model m, double value);
/* Model::set_l2 (v1/ops/regularizers/l2.cpp L:31-66). */
int ref_set_l2(ref_model m, double value);
int ref_set_clip_gradient(ref_model m, int use, double value);
int ref_set_constraint_recurrent_weight(ref_model m, size_t layer, double lower, double upper);
/* Model::save_params + save_spec_params, Model::load (v1/learner/save.cpp, load.cpp). */
int ref_save(ref_model m, const char *path_params, const char *path_spec);
int ref_load(ref_model m, const char *path_params, const char *path_spec);
int ref_set_propagation(ref_model m, int state);
int ref_set_accu_fn(ref_model m, int fn);
int ref_set_accu_var(ref_model m, double v);
int ref_compute_loss(ref_model m, size_t batch, const float *Y);
double ref_get_accu(ref_model m, size_t rows_total);
int ref_seed_uout(ref_model m, unsigned seed);
int ref_uout_draws(unsigned seed, size_t n_layers, size_t rows, const size_t *widths,
                   const float *betas, float *out);
int ref_set_seq_w(ref_model m, size_t time_delays);
int ref_seed_weights(ref_model m, unsigned seed);
int ref_initialize_weights_with_glorot_uniform(ref_model m);

/* name: total_parameters, total_weights, total_bias, total_layers,
 * number_threads, batch_size, seq_w, n_inp, n_out, total_normalized_units. */
size_t ref_get_size(ref_model m, const char *name);
/* out[0..9] = type_layer, n_out, first_connection, last_connection,
 * first_bias, last_bias, type_normalization, type_dropout, type_group,
 * first norm-unit index (offset of the layer's gamma inside the scale block)
 */
int ref_layer_info(ref_model m, size_t layer, size_t *out);

/* name: parameters, derivatives (thread-0 copy), first_moment, second_moment,
 * second_moment_hat, mask_regularized. */
int ref_get_array(ref_model m, const char *name, float *out, size_t n);
int ref_set_array(ref_model m, const char *name, const float *in, size_t n);
/* name: mean_average, variance_average, r_correction, d_correction, mean,
 * variance, scale, shift.  n = T * units. */
int ref_get_layer_norm(ref_model m, size_t layer, const char *name, float *out,
                       size_t n);
int ref_set_layer_norm(ref_model m, size_t layer, const char *name,
                       const float *in, size_t n);
int ref_set_dropout_mask(ref_model m, size_t layer, const uint8_t *mask,
                         size_t n);
/* Reseeds every ShakeDrop generator (Bernoulli and real, all threads). */
int ref_seed_shakedrop(ref_model m, unsigned seed);

/* The draws a serial (set_mp(0)) step makes from the ShakeDrop generators after
 * ref_seed_shakedrop(m, seed), replayed with copies of the reference's own
 * generator classes: forward, residual layers in order, per row one Bernoulli
 * draw and, if set, `width` draws of U(-1,1); backward, residual layers in
 * reverse, `width` draws of U(0,1) for every flagged row.  masks: [n_blocks,
 * rows]; forward/backward: [n_blocks, rows, width] (rows not flagged hold 1). */
int ref_shakedrop_draws(unsigned seed, size_t n_blocks, size_t rows, size_t width,
                        const float *probabilities, uint8_t *masks, float *forward,
                        float *backward);

int ref_train_begin(ref_model m, size_t batch);
/* X: [batch, seq_w * n_inp] row-major, Y: [batch, seq_w * n_out]. */
int ref_forward_pass(ref_model m, size_t batch, const float *X);
int ref_compute_error(ref_model m, size_t batch, const float *Y);
int ref_backward_pass(ref_model m, size_t batch);
int ref_update_derivatives(ref_model m, size_t batch);
int ref_merge_derivatives(ref_model m);
double ref_get_loss(ref_model m);
int ref_reset_loss(ref_model m);
int ref_update_weights(ref_model m, size_t batch, size_t training_size);
/* forward, error, backward, gradient accumulation in one OpenMP region as
 * Driver::train_mp does (lib/deep-learning/drivers/driver.cpp L:227-266);
 * writes the batch loss before the update to *loss. */
int ref_train_step(ref_model m, size_t batch, const float *X, const float *Y,
                   double *loss);
/* Compact copy [seq_w, batch, n_out(layer)] of layer->ptr_array_outputs. */
int ref_get_layer_outputs(ref_model m, size_t layer, size_t batch, float *out);
/* which: 0 = neuron errors (delta after normalisation backward),
 *        1 = derivative_outputs. */
int ref_get_layer_errors(ref_model m, size_t layer, size_t batch, int which,
                         float *out);

/* Flat-array optimizer update, no model graph: runs the reference's
 * Update_Parameters__<rule> on caller arrays of n elements for `steps` steps,
 * refilling the gradient from grad_fill (n floats) before each step.  Returns
 * seconds spent inside the update calls (for the CPU baseline). */
double ref_optimizer_sweep(int optimizer, size_t n, int steps, int use_mp,
                           float *p, const float *grad_fill, float *m, float *v,
                           float *vhat, const double *hparams /*lr,b1,b2,eps,gamma,final_lr,lgamma*/);

#ifdef __cplusplus
}
#endif
