/* Test infrastructure, not product code.
 *
 * The binding INTEGRATION.md describes, as code: DL::v1::Model::set_b200 replays
 * the construction the host Model went through on a dlb_model, and the hooks of
 * dropin_glue.h route the step entry points (forward_pass, compute_error,
 * backward_pass, update_derivatives, merge_mp_derivatives, update_weights_mp /
 * _st, get_loss, reset_loss) to the library's entry points of the same names.
 * Compiled only into oracle/_ref/libdlref_dropin.so, against the patched copy of
 * the reference's model.hpp that oracle/dropin_patch.py writes.  Scope: stacks of
 * fully connected layers (the reference's switch Model::set_cu,
 * v1/learner/model.cpp L:2300-2351, is the model for this function).
 */
#include "pch.hpp"

#include "deep-learning/data/enum/env.hpp"
#include "deep-learning/io/logger.hpp"
#include "deep-learning/v1/learner/model.hpp"

#include <omp.h>

#include <cstdio>
#include <vector>

#include "dlb200.h"
#include "dropin_glue.h"

using namespace DL;
using namespace DL::v1;

namespace {
dlb_model *lib_model(Model const *m) { return static_cast<dlb_model *>(m->b200_model); }

/* The reference's convention: log and go on (void entry points cannot fail). */
bool ok(dlb_status st, char const *what) {
  if (st == DLB_OK) return true;
  std::fprintf(stderr, "dlb drop-in: %s: %s [%s]\n", what, dlb_status_string(st), dlb_last_error());
  return false;
}
}  // namespace

bool Model::set_b200(bool const on, int const device) {
  if (!on) {
    if (this->b200_model) dlb_model_destroy(lib_model(this));
    if (this->b200_ctx) dlb_ctx_destroy(static_cast<dlb_ctx *>(this->b200_ctx));
    this->b200_model = this->b200_ctx = nullptr;
    this->b200_on = false;
    return true;
  }
  dlb_ctx *ctx = nullptr;
  dlb_model *lm = nullptr;
  if (!ok(dlb_ctx_create(&ctx, device), "dlb_ctx_create")) return false;
  if (!ok(dlb_model_create(&lm, ctx), "dlb_model_create")) return false;
  /* Replay the construction the host Model already went through. */
  std::vector<int> types;
  std::vector<size_t> units;
  for (Layer const *l = this->ptr_array_layers; l != this->ptr_last_layer; ++l) {
    types.push_back(static_cast<int>(l->type_layer));
    units.push_back(*l->ptr_number_outputs);
  }
  bool good = ok(dlb_model_compile(lm, types.size(), this->seq_w, static_cast<int>(this->type), types.data(),
                                   units.data()),
                 "compile");
  for (size_t i = 1; good && i != this->total_layers; ++i) {
    Layer const &l = this->ptr_array_layers[i];
    good = good && ok(dlb_model_set_layer_activation_function(
                          lm, i, static_cast<int>(*l.ptr_array_AF_units->ptr_type_activation_function)),
                      "set_layer_activation_function");
  }
  for (size_t i = 0; good && i != this->total_layers; ++i) {
    Layer const &l = this->ptr_array_layers[i];
    if (l.type_normalization != LAYER_NORM::NONE)
      good = good && ok(dlb_model_set_layer_normalization(lm, i, static_cast<int>(l.type_normalization)),
                        "Set__Layer_Normalization");
  }
  for (size_t i = 0; good && i != this->total_layers; ++i) {
    Layer const &l = this->ptr_array_layers[i];
    if (l.type_dropout != LAYER_DROPOUT::NONE)
      good = good && ok(dlb_model_set_dropout(lm, i, static_cast<int>(l.type_dropout), l.dropout_values[0], 0),
                        "set_dropout");
  }
  if (good) {
    dlb_model_set_normalization_momentum_average(lm, this->normalization_momentum_average);
    dlb_model_set_normalization_epsilon(lm, this->normalization_epsilon);
    dlb_model_set_brn_r_correction_maximum(lm, this->batch_renormalization_r_correction_maximum);
    dlb_model_set_brn_d_correction_maximum(lm, this->batch_renormalization_d_correction_maximum);
    good = ok(dlb_model_set_loss_fn(lm, static_cast<int>(this->type_loss_function)), "set_loss_fn") &&
           ok(dlb_model_set_optimizer(lm, static_cast<int>(this->type_optimizer_function)), "set_optimizer");
  }
  if (good) {
#define FIELD(f) dlb_model_set_hparam(lm, #f, static_cast<double>(this->f));
    FIELD(adam_learning_rate) FIELD(adam_beta1) FIELD(adam_beta2) FIELD(adam_epsilon) FIELD(adam_gamma)
    FIELD(adam_previous_beta2) FIELD(learning_rate_final) FIELD(learning_gamma) FIELD(learning_rate)
    FIELD(learning_momentum) FIELD(optimizer_time_step) FIELD(epoch_time_step)
#undef FIELD
    dlb_model_set_hparam(lm, "use_adam_bias_correction", this->use_adam_bias_correction ? 1.0 : 0.0);
    dlb_model_set_hparam(lm, "use_nesterov", this->use_nesterov ? 1.0 : 0.0);
    dlb_model_set_hparam(lm, "use_normalized_weight_decay", this->use_normalized_weight_decay ? 1.0 : 0.0);
    dlb_model_set_weight_decay(lm, this->weight_decay);
    dlb_model_set_clip_gradient(lm, this->use_clip_gradient ? 1 : 0, this->clip_gradient);
    if (this->n_time_delay) dlb_model_set_seq_w(lm, this->n_time_delay);
    dlb_model_set_max_batch_size(lm, this->batch_size);
    good = ok(dlb_model_set_array(lm, "parameters", this->ptr_array_parameters, this->total_parameters),
              "parameters to the device");
  }
  if (!good) {
    dlb_model_destroy(lm);
    dlb_ctx_destroy(ctx);
    return false;
  }
  this->b200_ctx = ctx;
  this->b200_model = lm;
  this->b200_on = true;
  return true;
}

namespace dlb_dropin {

bool first_thread() { return omp_get_thread_num() == 0; }

void forward(Model *m, size_t rows, float const *const *Xm) {
  dlb_model *lm = lib_model(m);
  /* Masks drawn by Model::Dropout_Bernoulli (or written by a test) live in the
   * host Model; hand them over before they are used. */
  for (size_t i = 0; i + 1 < m->total_layers; ++i) {
    Layer const &l = m->ptr_array_layers[i];
    if ((l.type_dropout == LAYER_DROPOUT::BERNOULLI || l.type_dropout == LAYER_DROPOUT::BERNOULLI_INVERTED) &&
        l.ptr_array__mask__dropout__bernoulli) {
      size_t const n = m->seq_w * *l.ptr_number_outputs;
      std::vector<uint8_t> mask(n);
      for (size_t k = 0; k < n; ++k) mask[k] = l.ptr_array__mask__dropout__bernoulli[k] ? 1 : 0;
      ok(dlb_model_set_dropout_mask(lm, i, mask.data(), n), "set_dropout_mask");
    }
  }
  dlb_model_set_propagation(lm, m->type_state_propagation == PROPAGATION::TRAINING ? DLB_PROPAGATION_TRAINING
                                                                                  : DLB_PROPAGATION_INFERENCE);
  ok(dlb_model_forward_pass(lm, rows, Xm), "forward_pass");
}
void error(Model *m, size_t rows, float const *const *Ym) { ok(dlb_model_compute_error(lib_model(m), rows, Ym), "compute_error"); }
void backward(Model *m, size_t rows) { ok(dlb_model_backward_pass(lib_model(m), rows), "backward_pass"); }
void derivatives(Model *m, size_t rows) { ok(dlb_model_update_derivatives(lib_model(m), rows), "update_derivatives"); }
void merge(Model *m) { ok(dlb_model_merge_derivatives(lib_model(m)), "merge_derivatives"); }
void update(Model *m, size_t rows, size_t training_size) {
  dlb_model *lm = lib_model(m);
  if (!ok(dlb_model_update_weights(lm, rows, training_size), "update_weights")) return;
  /* Copy__Parameters__Device_To_Host: the host mirror follows every update here,
   * so that Model::save_params and the tests read current weights. */
  ok(dlb_model_get_array(lm, "parameters", m->ptr_array_parameters, m->total_parameters), "parameters to the host");
  m->optimizer_time_step = static_cast<real>(dlb_model_get_hparam(lm, "optimizer_time_step"));
}
double loss(Model const *m) {
  double v = 1.0;
  ok(dlb_model_get_loss(lib_model(m), &v), "get_loss");
  return v;
}
void reset_loss(Model *m) { ok(dlb_model_reset_loss(lib_model(m)), "reset_loss"); }

}  // namespace dlb_dropin

extern "C" int ref_set_b200(void *handle_model, int on, int device) {
  /* The harness's handle starts with the Model (ref_harness.cpp, struct Handle). */
  return static_cast<Model *>(handle_model)->set_b200(on != 0, device) ? 0 : -1;
}
