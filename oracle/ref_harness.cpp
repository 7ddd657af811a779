/* Test infrastructure, not product code.
 *
 * Driver around the reference library's DL::v1::Model (see ref_harness.h).
 * This file is original code; it includes the reference's headers from where
 * they lie and is linked with objects compiled from the reference's own
 * sources.  The step sequence mirrors Driver::train / Driver::train_mp
 * (lib/deep-learning/drivers/driver.cpp L:107-160, L:227-266) except that the
 * dropout masks are written by the caller instead of being drawn from a
 * clock-seeded generator.
 */
#include "pch.hpp"

#include "deep-learning/data/enum/env.hpp"
#include "deep-learning/io/logger.hpp"
#include "deep-learning/v1/learner/model.hpp"

#include <omp.h>

#include <chrono>
#include <iostream>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "ref_harness.h"

using namespace DL;
using namespace DL::v1;

namespace {
struct Handle {
  Model model;
  std::vector<const float *> rows_x, rows_y;
  bool training_started = false;
};

void ensure_logger() {
  /* ERR()/ASSERT_MSG dereference the global logger. */
  static std::unique_ptr<Logger> lg;
  if (!lg) {
    lg = std::make_unique<Logger>(LOGLEVEL::FATAL);
    /* Dist::Bernoulli::probability() logs a FATAL line on every call (its
     * assertion is `p >= 0 && p < 0`, ops/distributions/bernoulli.cpp L:56);
     * the logger writes to std::wcout, which is silenced here. */
    std::wcout.setstate(std::ios_base::failbit);
  }
}

inline Handle *H(ref_model m) { return static_cast<Handle *>(m); }

Layer *layer_at(Handle *h, size_t i) {
  if (i >= h->model.total_layers) return nullptr;
  return h->model.ptr_array_layers + i;
}

size_t layer_norm_units(Layer const *l) {
  return static_cast<size_t>(l->ptr_last_normalized_unit -
                             l->ptr_array_normalized_units);
}

void make_rows(std::vector<const float *> &rows, const float *base, size_t n,
               size_t stride) {
  rows.resize(n);
  for (size_t i = 0; i < n; ++i) rows[i] = base + i * stride;
}
}  // namespace

extern "C" {

ref_model ref_model_create(void) {
  ensure_logger();
  return new Handle;
}

void ref_model_destroy(ref_model m) { delete H(m); }

int ref_compile(ref_model m, size_t n_layers, size_t seq_w, int model_type,
                const int *layer_types, const size_t *layer_units,
                size_t allowable_memory) {
  std::vector<Layer_Parameters> ls(n_layers);
  for (size_t i = 0; i < n_layers; ++i) {
    ls[i].type_layer = static_cast<LAYER::TYPE>(layer_types[i]);
    ls[i].unit_parameters[0] = layer_units[i];
  }
  return H(m)->model.compile(n_layers, seq_w,
                             static_cast<MODEL::TYPE>(model_type), ls.data(),
                             allowable_memory)
             ? 0
             : -1;
}

/* compile() with the second unit parameter of a layer (cells per block of an
 * LSTM layer; Layer_Parameters::unit_parameters[1]). */
int ref_compile2(ref_model m, size_t n_layers, size_t seq_w, int model_type, const int *layer_types,
                 const size_t *layer_units, const size_t *layer_units2, size_t allowable_memory) {
  std::vector<Layer_Parameters> ls(n_layers);
  for (size_t i = 0; i < n_layers; ++i) {
    ls[i].type_layer = static_cast<LAYER::TYPE>(layer_types[i]);
    ls[i].unit_parameters[0] = layer_units[i];
    ls[i].unit_parameters[1] = layer_units2[i];
  }
  return H(m)->model.compile(n_layers, seq_w, static_cast<MODEL::TYPE>(model_type), ls.data(), allowable_memory)
             ? 0
             : -1;
}

int ref_set_layer_activation_function(ref_model m, size_t layer, int af) {
  return H(m)->model.set_layer_activation_function(
             layer, static_cast<ACTIVATION::TYPE>(af))
             ? 0
             : -1;
}

int ref_set_layer_normalization(ref_model m, size_t layer, int norm) {
  return H(m)->model.Set__Layer_Normalization(
             layer, static_cast<LAYER_NORM::TYPE>(norm))
             ? 0
             : -1;
}

int ref_set_dropout(ref_model m, size_t layer, int type, float value0,
                    int scale_weights) {
  real values[3] = {value0, 0, 0};
  return H(m)->model.set_dropout(layer, static_cast<LAYER_DROPOUT::TYPE>(type),
                                 values, scale_weights != 0)
             ? 0
             : -1;
}

int ref_set_normalization_momentum_average(ref_model m, float v) {
  return H(m)->model.Set__Normalization_Momentum_Average(v) ? 0 : -1;
}
int ref_set_normalization_epsilon(ref_model m, float v) {
  return H(m)->model.Set__Normalization_Epsilon(v) ? 0 : -1;
}
int ref_set_brn_r_correction_maximum(ref_model m, float v) {
  return H(m)->model.Set__Batch_Renormalization_r_Correction_Maximum(v) ? 0
                                                                         : -1;
}
int ref_set_brn_d_correction_maximum(ref_model m, float v) {
  return H(m)->model.Set__Batch_Renormalization_d_Correction_Maximum(v) ? 0
                                                                         : -1;
}

int ref_set_loss_fn(ref_model m, int loss) {
  H(m)->model.set_loss_fn(static_cast<LOSS_FN::TYPE>(loss));
  /* The accuracy function is off the compared path; any valid value. */
  H(m)->model.set_accu_fn(loss == LOSS_FN::CROSS_ENTROPY
                              ? ACCU_FN::CROSS_ENTROPY
                              : ACCU_FN::DISTANCE);
  return 0;
}

int ref_set_optimizer(ref_model m, int optimizer) {
  H(m)->model.set_optimizer(static_cast<OPTIMIZER::TYPE>(optimizer));
  return 0;
}

#define HPARAM_LIST(X)            \
  X(adam_learning_rate)           \
  X(adam_beta1)                   \
  X(adam_beta2)                   \
  X(adam_epsilon)                 \
  X(adam_gamma)                   \
  X(adam_previous_beta2)          \
  X(learning_rate_final)          \
  X(learning_rate)                \
  X(learning_momentum)            \
  X(learning_gamma)               \
  X(weight_decay)                 \
  X(optimizer_time_step)          \
  X(epoch_time_step)

int ref_set_hparam(ref_model m, const char *name, double value) {
  Model &M = H(m)->model;
  std::string n(name);
#define X(f)                        \
  if (n == #f) {                    \
    M.f = static_cast<real>(value); \
    return 0;                       \
  }
  HPARAM_LIST(X)
#undef X
  if (n == "use_adam_bias_correction") {
    M.use_adam_bias_correction = value != 0.0;
    return 0;
  }
  if (n == "use_nesterov") {
    M.use_nesterov = value != 0.0;
    return 0;
  }
  if (n == "use_normalized_weight_decay") {
    M.use_normalized_weight_decay = value != 0.0;
    return 0;
  }
  if (n == "pct_threads") return M.Set__Maximum_Thread_Usage(value) ? 0 : -1;
  return -1;
}

double ref_get_hparam(ref_model m, const char *name) {
  Model &M = H(m)->model;
  std::string n(name);
#define X(f) \
  if (n == #f) return static_cast<double>(M.f);
  HPARAM_LIST(X)
#undef X
  if (n == "use_adam_bias_correction") return M.use_adam_bias_correction;
  return -1.0;
}

int ref_set_max_batch_size(ref_model m, size_t b) {
  return H(m)->model.set_max_batch_size(b) ? 0 : -1;
}
int ref_set_mp(ref_model m, int use_mp) {
  return H(m)->model.set_mp(use_mp != 0) ? 0 : -1;
}
int ref_set_weight_decay(ref_model m, double value) {
  return H(m)->model.set_weight_decay(static_cast<real>(value)) ? 0 : -1;
}
int ref_set_l2(ref_model m, double value) {
  return H(m)->model.set_l2(static_cast<real>(value)) ? 0 : -1;
}
int ref_set_clip_gradient(ref_model m, int use, double value) {
  H(m)->model.set_clip_gradient(use != 0);
  return H(m)->model.set_clip_gradient(static_cast<real>(value)) ? 0 : -1;
}
int ref_set_constraint_recurrent_weight(ref_model m, size_t layer, double lower, double upper) {
  return H(m)->model.Set__Regularization__Constraint_Recurrent_Weight(layer, static_cast<real>(lower),
                                                                      static_cast<real>(upper))
             ? 0
             : -1;
}
int ref_save(ref_model m, const char *path_params, const char *path_spec) {
  std::string a(path_params), b(path_spec);
  Model &M = H(m)->model;
  if (!M.save_params(std::wstring(a.begin(), a.end()))) return -1;
  return M.save_spec_params(std::wstring(b.begin(), b.end())) ? 0 : -2;
}
int ref_load(ref_model m, const char *path_params, const char *path_spec) {
  std::string a(path_params), b(path_spec);
  return H(m)->model.load(std::wstring(a.begin(), a.end()), std::wstring(b.begin(), b.end()),
                          static_cast<size_t>(8) << 30)
             ? 0
             : -1;
}
int ref_set_seq_w(ref_model m, size_t time_delays) {
  return H(m)->model.set_seq_w(time_delays) ? 0 : -1;
}
int ref_seed_weights(ref_model m, unsigned seed) {
  H(m)->model.real_gen.seed(seed);
  return 0;
}
int ref_initialize_weights_with_glorot_uniform(ref_model m) {
  H(m)->model.initialize_weights_with_glorot_uniform();
  return 0;
}

size_t ref_get_size(ref_model m, const char *name) {
  Model &M = H(m)->model;
  std::string n(name);
#define X(f) \
  if (n == #f) return M.f;
  X(total_parameters)
  X(total_weights)
  X(total_bias)
  X(total_layers)
  X(number_threads)
  X(batch_size)
  X(seq_w)
  X(n_time_delay)
  X(n_inp)
  X(n_out)
  X(total_normalized_units)
  X(total_parameters_allocated)
#undef X
  return static_cast<size_t>(-1);
}

int ref_layer_info(ref_model m, size_t layer, size_t *out) {
  Handle *h = H(m);
  Layer *l = layer_at(h, layer);
  if (!l) return -1;
  out[0] = static_cast<size_t>(l->type_layer);
  out[1] = l->ptr_number_outputs ? *l->ptr_number_outputs : 0;
  out[2] = l->ptr_first_connection_index ? *l->ptr_first_connection_index : 0;
  out[3] = l->ptr_last_connection_index ? *l->ptr_last_connection_index : 0;
  out[4] = l->first_bias_connection_index;
  out[5] = l->last_bias_connection_index;
  out[6] = static_cast<size_t>(l->type_normalization);
  out[7] = static_cast<size_t>(l->type_dropout);
  out[8] = static_cast<size_t>(l->type_group);
  out[9] = 0;
  if (layer_norm_units(l) != 0 &&
      h->model.ptr_array_normalized_batch_units_scales != nullptr)
    out[9] = static_cast<size_t>(
        l->ptr_array_normalized_units->normalized_batch_units.ptr_scale -
        h->model.ptr_array_normalized_batch_units_scales);
  return 0;
}

static real *named_array(Model &M, const std::string &n) {
  if (n == "parameters") return M.ptr_array_parameters;
  if (n == "derivatives") return M.ptr_array_derivatives_parameters;
  if (n == "first_moment") return M.ptr_array_previous_biased_first_moment;
  if (n == "second_moment") return M.ptr_array_previous_biased_second_moment;
  if (n == "second_moment_hat")
    return M.ptr_array_previous_biased_second_moment_hat;
  if (n == "mask_regularized") return M.ptr_array_mask_regularized_parameters;
  return nullptr;
}

int ref_get_array(ref_model m, const char *name, float *out, size_t n) {
  real *p = named_array(H(m)->model, name);
  if (!p || n > H(m)->model.total_parameters) return -1;
  std::memcpy(out, p, n * sizeof(float));
  return 0;
}

int ref_set_array(ref_model m, const char *name, const float *in, size_t n) {
  real *p = named_array(H(m)->model, name);
  if (!p || n > H(m)->model.total_parameters) return -1;
  std::memcpy(p, in, n * sizeof(float));
  return 0;
}

static real *norm_field(Normalized_batch_unit &u, const std::string &n) {
  if (n == "mean_average") return u.ptr_mean_average;
  if (n == "variance_average") return u.ptr_variance_average;
  if (n == "r_correction") return u.ptr_r_correction;
  if (n == "d_correction") return u.ptr_d_correction;
  if (n == "mean") return u.ptr_array_means;
  if (n == "variance") return u.ptr_array_variances;
  if (n == "scale") return u.ptr_scale;
  if (n == "shift") return u.ptr_shift;
  return nullptr;
}

/* Per-unit statistics are stored [T][units_total] with the unit's own pointer
 * addressing t = 0; element t of a unit is units_total floats further
 * (lib/deep-learning/v1/learner/fwp_mp.cpp L:4666-4718). */
static int layer_norm_io(ref_model m, size_t layer, const char *name,
                         float *out, const float *in, size_t n) {
  Handle *h = H(m);
  Layer *l = layer_at(h, layer);
  if (!l) return -1;
  size_t const units = layer_norm_units(l);
  if (units == 0) return -1;
  std::string nm(name);
  bool const per_t = !(nm == "scale" || nm == "shift");
  size_t const T = per_t ? h->model.seq_w : 1;
  if (n != T * units) return -1;
  /* A layer's statistics are [T][units of the layer], the unit's own pointer
   * addressing t = 0 (v1/learner/allocate.cpp L:1348-1356). */
  size_t const stride = units;
  for (size_t u = 0; u < units; ++u) {
    real *p = norm_field(l->ptr_array_normalized_units[u].normalized_batch_units,
                         nm);
    if (!p) return -1;
    for (size_t t = 0; t < T; ++t) {
      if (out) out[t * units + u] = p[t * stride];
      if (in) p[t * stride] = in[t * units + u];
    }
  }
  return 0;
}

int ref_get_layer_norm(ref_model m, size_t layer, const char *name, float *out,
                       size_t n) {
  return layer_norm_io(m, layer, name, out, nullptr, n);
}
int ref_set_layer_norm(ref_model m, size_t layer, const char *name,
                       const float *in, size_t n) {
  return layer_norm_io(m, layer, name, nullptr, in, n);
}

int ref_set_dropout_mask(ref_model m, size_t layer, const uint8_t *mask,
                         size_t n) {
  Layer *l = layer_at(H(m), layer);
  if (!l || !l->ptr_array__mask__dropout__bernoulli) return -1;
  for (size_t i = 0; i < n; ++i)
    l->ptr_array__mask__dropout__bernoulli[i] = mask[i] != 0;
  return 0;
}

int ref_seed_shakedrop(ref_model m, unsigned seed) {
  Model &M = H(m)->model;
  if (!M.ptr_array_Class_Generator_Bernoulli_ShakeDrop ||
      !M.ptr_array_Class_Generator_Real_ShakeDrop)
    return -1;
  for (size_t t = 0; t < M.number_threads; ++t) {
    M.ptr_array_Class_Generator_Bernoulli_ShakeDrop[t].seed(
        seed + static_cast<unsigned>(2 * t));
    M.ptr_array_Class_Generator_Real_ShakeDrop[t].seed(
        seed + static_cast<unsigned>(2 * t + 1));
  }
  return 0;
}

int ref_shakedrop_draws(unsigned seed, size_t n_blocks, size_t rows, size_t width,
                        const float *probabilities, uint8_t *masks, float *forward,
                        float *backward) {
  ensure_logger();
  /* Same seeds as ref_seed_shakedrop gives thread 0. */
  Dist::Bernoulli bern;
  Dist::Real real_gen;
  bern.seed(seed);
  real_gen.seed(seed + 1u);
  for (size_t i = 0; i < n_blocks * rows * width; ++i) forward[i] = backward[i] = 1.0f;
  for (size_t b = 0; b < n_blocks; ++b) {
    bern.probability(probabilities[b]);
    real_gen.range(-1_r, 1_r);
    for (size_t r = 0; r < rows; ++r) {
      bool const hit = bern();
      masks[b * rows + r] = hit ? 1 : 0;
      if (hit)
        for (size_t k = 0; k < width; ++k) forward[(b * rows + r) * width + k] = real_gen();
    }
  }
  for (size_t b = n_blocks; b-- > 0;) {
    real_gen.range(0_r, 1_r);
    for (size_t r = 0; r < rows; ++r)
      if (masks[b * rows + r])
        for (size_t k = 0; k < width; ++k) backward[(b * rows + r) * width + k] = real_gen();
  }
  return 0;
}

int ref_seed_uout(ref_model m, unsigned seed) {
  Model &M = H(m)->model;
  if (!M.ptr_array_Class_Generator_Real_Uout) return -1;
  for (size_t t = 0; t < M.number_threads; ++t)
    M.ptr_array_Class_Generator_Real_Uout[t].seed(seed + static_cast<unsigned>(t));
  return 0;
}

int ref_uout_draws(unsigned seed, size_t n_layers, size_t rows, const size_t *widths,
                   const float *betas, float *out) {
  ensure_logger();
  /* What a serial forward pass draws after ref_seed_uout(seed): layer by
   * layer, rows * width values of U(-beta, beta) each. */
  Dist::Real gen;
  gen.seed(seed);
  size_t o = 0;
  for (size_t l = 0; l < n_layers; ++l) {
    gen.range(-static_cast<real>(betas[l]), static_cast<real>(betas[l]));
    for (size_t i = 0; i < rows * widths[l]; ++i) out[o++] = gen();
  }
  return 0;
}

int ref_train_begin(ref_model m, size_t batch) {
  Handle *h = H(m);
  Model &M = h->model;
  if (M.ptr_array_derivatives_parameters == nullptr) M.clear_training_arrays();
  M.type_state_propagation = PROPAGATION::TRAINING;
  if (!M.update_mem_batch_size(batch)) return -1;
  if (M.use_mp && M.is_mp_initialized) {
    if (!M.update_mem_thread_size(batch)) return -1;
    omp_set_num_threads(static_cast<int>(M.number_threads));
  }
  h->training_started = true;
  return 0;
}

int ref_forward_pass(ref_model m, size_t batch, const float *X) {
  Handle *h = H(m);
  Model &M = h->model;
  make_rows(h->rows_x, X, batch, M.seq_w * M.n_inp);
  if (M.use_mp && M.is_mp_initialized) {
#pragma omp parallel
    M.forward_pass(batch, h->rows_x.data());
  } else {
    M.forward_pass(batch, h->rows_x.data());
  }
  return 0;
}

int ref_compute_error(ref_model m, size_t batch, const float *Y) {
  Handle *h = H(m);
  Model &M = h->model;
  make_rows(h->rows_y, Y, batch, M.seq_w * M.n_out);
  if (M.use_mp && M.is_mp_initialized) {
#pragma omp parallel
    M.compute_error(batch, h->rows_y.data());
  } else {
    M.compute_error(batch, h->rows_y.data());
  }
  return 0;
}

/* Evaluation, as Driver::evalt (drivers/driver.cpp L:60-105, L:172-226): the
 * propagation state, the loss-only pass over the outputs of a forward pass,
 * the merge of the per-thread counters and the accuracy in percent. */
int ref_set_propagation(ref_model m, int state) {
  H(m)->model.type_state_propagation = static_cast<PROPAGATION::TYPE>(state);
  return 0;
}
int ref_set_accu_fn(ref_model m, int fn) {
  H(m)->model.set_accu_fn(static_cast<ACCU_FN::TYPE>(fn));
  return 0;
}
int ref_set_accu_var(ref_model m, double v) {
  H(m)->model.acc_var = static_cast<real>(v);
  return 0;
}
int ref_compute_loss(ref_model m, size_t batch, const float *Y) {
  Handle *h = H(m);
  Model &M = h->model;
  make_rows(h->rows_y, Y, batch, M.seq_w * M.n_out);
  if (M.use_mp && M.is_mp_initialized) {
#pragma omp parallel
    M.compute_loss(batch, h->rows_y.data());
  } else {
    M.compute_loss(batch, h->rows_y.data());
  }
  M.merge_mp_accu_loss();
  return 0;
}
double ref_get_accu(ref_model m, size_t rows_total) {
  Model &M = H(m)->model;
  M.n_acc_trial = rows_total * (M.seq_w - M.n_time_delay) *
                  (ACCU_FN::CROSS_ENTROPY == M.type_accuracy_function ? 1_UZ : M.n_out);
  return M.get_accu(ENV::NONE);
}

int ref_backward_pass(ref_model m, size_t batch) {
  Model &M = H(m)->model;
  if (M.use_mp && M.is_mp_initialized) {
#pragma omp parallel
    M.backward_pass(batch);
  } else {
    M.backward_pass(batch);
  }
  return 0;
}

int ref_update_derivatives(ref_model m, size_t batch) {
  Model &M = H(m)->model;
  if (M.use_mp && M.is_mp_initialized) {
#pragma omp parallel
    M.update_derivatives(batch, M.ptr_array_layers + 1, M.ptr_last_layer);
  } else {
    M.update_derivatives(batch, M.ptr_array_layers + 1, M.ptr_last_layer);
  }
  return 0;
}

int ref_merge_derivatives(ref_model m) {
  Model &M = H(m)->model;
  if (M.use_mp && M.is_mp_initialized) {
    M.merge_mp_derivatives(0, M.total_parameters);
    M.merge_mp_accu_loss();
  }
  return 0;
}

double ref_get_loss(ref_model m) { return H(m)->model.get_loss(ENV::NONE); }

int ref_reset_loss(ref_model m) {
  H(m)->model.reset_loss();
  return 0;
}

int ref_update_weights(ref_model m, size_t batch, size_t training_size) {
  Model &M = H(m)->model;
  if (M.use_mp && M.is_mp_initialized)
    M.update_weights_mp(batch, training_size);
  else
    M.update_weights_st(batch, training_size);
  return 0;
}

int ref_train_step(ref_model m, size_t batch, const float *X, const float *Y,
                   double *loss) {
  Handle *h = H(m);
  Model &M = h->model;
  if (!h->training_started && ref_train_begin(m, batch) != 0) return -1;
  make_rows(h->rows_x, X, batch, M.seq_w * M.n_inp);
  make_rows(h->rows_y, Y, batch, M.seq_w * M.n_out);
  M.reset_loss();
  if (M.use_mp && M.is_mp_initialized) {
#pragma omp parallel
    {
      M.forward_pass(batch, h->rows_x.data());
      M.compute_error(batch, h->rows_y.data());
      M.backward_pass(batch);
      M.update_derivatives(batch, M.ptr_array_layers + 1, M.ptr_last_layer);
    }
    M.merge_mp_derivatives(0, M.total_parameters);
    M.merge_mp_accu_loss();
    if (loss) *loss = M.get_loss(ENV::NONE);
    M.update_weights_mp(batch, batch);
  } else {
    M.forward_pass(batch, h->rows_x.data());
    M.compute_error(batch, h->rows_y.data());
    M.backward_pass(batch);
    M.update_derivatives(batch, M.ptr_array_layers + 1, M.ptr_last_layer);
    if (loss) *loss = M.get_loss(ENV::NONE);
    M.update_weights_st(batch, batch);
  }
  return 0;
}

static int copy_tbh(Model &M, const real *src, size_t batch, size_t H_,
                    float *out) {
  if (!src) return -1;
  size_t const Bbar = M.batch_size, T = M.seq_w;
  for (size_t t = 0; t < T; ++t)
    std::memcpy(out + t * batch * H_, src + t * Bbar * H_,
                batch * H_ * sizeof(float));
  return 0;
}

int ref_get_layer_outputs(ref_model m, size_t layer, size_t batch, float *out) {
  Handle *h = H(m);
  Layer *l = layer_at(h, layer);
  if (!l) return -1;
  return copy_tbh(h->model, l->ptr_array_outputs, batch, *l->ptr_number_outputs,
                  out);
}

int ref_get_layer_errors(ref_model m, size_t layer, size_t batch, int which,
                         float *out) {
  Handle *h = H(m);
  Layer *l = layer_at(h, layer);
  if (!l) return -1;
  const real *src = nullptr;
  if (which == 0)
    src = l->ptr_array_neuron_units ? l->ptr_array_neuron_units->ptr_array_errors
                                    : nullptr;
  else
    src = l->ptr_array_derivative_outputs;
  return copy_tbh(h->model, src, batch, *l->ptr_number_outputs, out);
}

double ref_optimizer_sweep(int optimizer, size_t n, int steps, int use_mp,
                           float *p, const float *grad_fill, float *mm,
                           float *vv, float *vhat, const double *hp) {
  ensure_logger();
  auto M = std::make_unique<Model>();
  std::vector<float> g(n);
  M->total_parameters = n;
  M->ptr_array_parameters = p;
  M->ptr_array_derivatives_parameters = g.data();
  M->ptr_array_previous_biased_first_moment = mm;
  M->ptr_array_previous_biased_second_moment = vv;
  M->ptr_array_previous_biased_second_moment_hat = vhat;
  M->adam_learning_rate = static_cast<real>(hp[0]);
  M->adam_beta1 = static_cast<real>(hp[1]);
  M->adam_beta2 = static_cast<real>(hp[2]);
  M->adam_epsilon = static_cast<real>(hp[3]);
  M->adam_gamma = static_cast<real>(hp[4]);
  M->learning_rate_final = static_cast<real>(hp[5]);
  M->learning_gamma = static_cast<real>(hp[6]);
  M->weight_decay = 0;
  M->use_mp = use_mp != 0;
  M->is_mp_initialized = use_mp != 0;
  if (use_mp) {
    M->number_threads = static_cast<size_t>(omp_get_num_procs());
    omp_set_num_threads(static_cast<int>(M->number_threads));
  }
  double seconds = 0.0;
  int rc = 0;
  for (int s = 0; s < steps && rc == 0; ++s) {
    std::memcpy(g.data(), grad_fill, n * sizeof(float));
    auto t0 = std::chrono::steady_clock::now();
    switch (optimizer) {
      case OPTIMIZER::ADAM: M->Update_Parameters__Adam(1, 1, 0, n); break;
      case OPTIMIZER::AMSGRAD: M->Update_Parameters__AMSGrad(1, 1, 0, n); break;
      case OPTIMIZER::ADABOUND:
        M->Update_Parameters__AdaBound(1, 1, 0, n);
        break;
      case OPTIMIZER::AMSBOUND:
        M->Update_Parameters__AMSBound(1, 1, 0, n);
        break;
      case OPTIMIZER::NOSADAM: M->Update_Parameters__NosAdam(1, 1, 0, n); break;
      default: rc = -1; break;
    }
    seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() -
                                             t0)
                   .count();
  }
  /* The arrays belong to the caller: detach them before ~Model frees. */
  M->ptr_array_parameters = nullptr;
  M->ptr_array_derivatives_parameters = nullptr;
  M->ptr_array_previous_biased_first_moment = nullptr;
  M->ptr_array_previous_biased_second_moment = nullptr;
  M->ptr_array_previous_biased_second_moment_hat = nullptr;
  M->total_parameters = 0;
  return rc == 0 ? seconds : -1.0;
}

}  // extern "C"
