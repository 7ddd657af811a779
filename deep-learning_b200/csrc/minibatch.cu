// The mini-batch loop around the training step, host side.
//
// ref: DL::v1::MiniBatch (v1/data/dataset/minibatch.cpp): Set__Desired_Data_Per_Batch
// (L:118-190: number of batches, the larger last batch), Shuffle (L:42-58: a
// Fisher-Yates pass from the end with std::mt19937 and
// std::uniform_int_distribution), Increment_Mini_Batch (L:192-248: the batch's
// rows as pointers into the data set) and train_mp (L:286-323: per batch one
// training step and update_weights(batch rows, rows of the data set), the mean
// of the batch losses, epoch_time_step + 1).
//
// The reference hands each batch to the model as an array of row pointers and
// waits for it.  Here batch k + 1 is gathered into page-locked memory and sent
// to the device (dlb_model_stage_batch) while batch k trains, so the copy is
// off the critical path; the loss of every batch is read as the reference reads
// it.  Host code only.
#include <string.h>

#include <algorithm>
#include <random>
#include <thread>
#include <vector>

#include "common.cuh"
#include "model.cuh"

using namespace dlb;

struct dlb_minibatch {
  dlb_model *model = nullptr;
  const float *const *Xm = nullptr, *const *Ym = nullptr;
  size_t n_data = 0, n_batch = 0, per_batch = 0, last_batch = 0;
  size_t width_x = 0, width_y = 0;
  bool shuffle = false;
  std::vector<size_t> order;   // MiniBatch::ptr_array_stochastic_index
  std::mt19937 gen;            // DistributionBase::p_generator_mt19937
  float *host_x[2] = {nullptr, nullptr}, *host_y[2] = {nullptr, nullptr};  // page-locked, last_batch rows each
  double accuracy = 0.0;       // mean of the batch accuracies of the last pass (percent)
};

namespace {

size_t rows_of(const dlb_minibatch *mb, size_t k) { return k + 1 != mb->n_batch ? mb->per_batch : mb->last_batch; }

// Rows of batch k into staging slot `slot`, by the host threads the model keeps.
void gather(dlb_minibatch *mb, size_t k, int slot) {
  const size_t first = k * mb->per_batch, rows = rows_of(mb, k);
  auto part = [&](size_t a, size_t b) {
    for (size_t r = a; r < b; ++r) {
      const size_t src = mb->order[first + r];
      memcpy(mb->host_x[slot] + r * mb->width_x, mb->Xm[src], mb->width_x * sizeof(float));
      memcpy(mb->host_y[slot] + r * mb->width_y, mb->Ym[src], mb->width_y * sizeof(float));
    }
  };
  const size_t bytes = rows * (mb->width_x + mb->width_y) * sizeof(float);
  if (bytes < (1u << 20)) {
    part(0, rows);
    return;
  }
  dlb_model *m = mb->model;
  if (!m->workers) {
    const unsigned hw = std::thread::hardware_concurrency();
    m->workers = new HostWorkers(std::min<size_t>(8, hw ? hw : 1) - 1);
  }
  const size_t parts = m->workers->size() * 4;
  const size_t per = (rows + parts - 1) / parts;
  m->workers->run(parts, [&](size_t i) { part(std::min(rows, i * per), std::min(rows, (i + 1) * per)); });
}

}  // namespace

extern "C" {

dlb_status dlb_minibatch_create(dlb_minibatch **out, dlb_model *model, const float *const *Xm,
                                const float *const *Ym, size_t n_examples, int use_shuffle,
                                size_t desired_per_batch, size_t max_batches, unsigned seed) {
  DLB_REQUIRE(out && model && Xm && Ym && n_examples > 0, "dlb_minibatch_create");
  DLB_REQUIRE(desired_per_batch > 0 && desired_per_batch <= n_examples,
              "dlb_minibatch_create: rows per batch must be in [1, rows of the data set]");
  // Set__Desired_Data_Per_Batch: floor(N / desired) batches, at most max_batches;
  // the last batch takes the remainder as the reference computes it, from the
  // fractional part of N / desired.
  const double batches_real = (double)n_examples / (double)desired_per_batch;
  size_t n_batch = (size_t)batches_real;
  if (max_batches != 0) n_batch = std::min(n_batch, max_batches);
  if (n_batch <= 1) {
    set_error("dlb_minibatch_create: %zu rows in batches of %zu give %zu batch(es); the reference asks for two or more",
              n_examples, desired_per_batch, n_batch);
    return DLB_ERR_INVALID;
  }
  dlb_minibatch *mb = new dlb_minibatch;
  mb->model = model;
  mb->Xm = Xm;
  mb->Ym = Ym;
  mb->n_data = n_examples;
  mb->n_batch = n_batch;
  mb->per_batch = desired_per_batch;
  mb->last_batch = desired_per_batch + (size_t)((batches_real - (double)n_batch) * (double)desired_per_batch);
  mb->shuffle = use_shuffle != 0;
  mb->order.resize(n_examples);
  for (size_t i = 0; i < n_examples; ++i) mb->order[i] = i;
  mb->gen.seed(seed);
  mb->width_x = model->seq_w * model->layers.front().units;
  mb->width_y = model->seq_w * model->layers.back().units;
  for (int s = 0; s < 2; ++s) {
    dlb_status st = dlb_host_alloc(reinterpret_cast<void **>(&mb->host_x[s]), mb->last_batch * mb->width_x * sizeof(float));
    if (st == DLB_OK)
      st = dlb_host_alloc(reinterpret_cast<void **>(&mb->host_y[s]), mb->last_batch * mb->width_y * sizeof(float));
    if (st != DLB_OK) {
      dlb_minibatch_destroy(mb);
      return st;
    }
  }
  *out = mb;
  return DLB_OK;
}

dlb_status dlb_minibatch_destroy(dlb_minibatch *mb) {
  if (!mb) return DLB_OK;
  // Every staged batch has been trained on when dlb_minibatch_train returns, so
  // no copy out of the staging buffers is left; the model is not touched here
  // (it may be gone already).
  for (int s = 0; s < 2; ++s) {
    if (mb->host_x[s]) dlb_host_free(mb->host_x[s]);
    if (mb->host_y[s]) dlb_host_free(mb->host_y[s]);
  }
  delete mb;
  return DLB_OK;
}

size_t dlb_minibatch_get_n_batch(const dlb_minibatch *mb) { return mb ? mb->n_batch : 0; }
size_t dlb_minibatch_examples_per_batch(const dlb_minibatch *mb) { return mb ? mb->per_batch : 0; }
size_t dlb_minibatch_examples_last_batch(const dlb_minibatch *mb) { return mb ? mb->last_batch : 0; }

dlb_status dlb_minibatch_set_shuffle(dlb_minibatch *mb, int use_shuffle) {
  DLB_REQUIRE(mb, "dlb_minibatch_set_shuffle");
  mb->shuffle = use_shuffle != 0;
  // MiniBatch::Set__Use__Shuffle: switching it off puts the rows back in order.
  if (!mb->shuffle)
    for (size_t i = 0; i < mb->n_data; ++i) mb->order[i] = i;
  return DLB_OK;
}

// MiniBatch::Shuffle.
dlb_status dlb_minibatch_shuffle(dlb_minibatch *mb) {
  DLB_REQUIRE(mb, "dlb_minibatch_shuffle");
  std::uniform_int_distribution<size_t> dist;
  for (size_t i = mb->n_data; i-- != 0;) {
    dist.param(std::uniform_int_distribution<size_t>::param_type(0, i));
    std::swap(mb->order[dist(mb->gen)], mb->order[i]);
  }
  return DLB_OK;
}

dlb_status dlb_minibatch_get_order(const dlb_minibatch *mb, size_t *out, size_t n) {
  DLB_REQUIRE(mb && out && n == mb->n_data, "dlb_minibatch_get_order");
  memcpy(out, mb->order.data(), n * sizeof(size_t));
  return DLB_OK;
}

// MiniBatch::train_mp: one pass over the data set.  *loss: mean of the batch
// losses.  With several ranks every rank walks its own shard with the same
// batch sizes; the step's exchanges make the batches global.
dlb_status dlb_minibatch_train(dlb_minibatch *mb, double *loss) {
  DLB_REQUIRE(mb && loss, "dlb_minibatch_train");
  dlb_model *m = mb->model;
  if (mb->shuffle) DLB_TRY(dlb_minibatch_shuffle(mb));
  const size_t world = (size_t)std::max(1, dlb_comm_world(m->ctx));
  const size_t saved_training = m->training_size, saved_global = m->global_rows;
  DLB_TRY(dlb_model_set_training_size(m, mb->n_data * world));  // update_weights_mp(rows of the batch, rows of the data set)
  DLB_TRY(dlb_model_set_loss_lag(m, 0));
  const bool saved_accuracy = m->training_accuracy;
  m->training_accuracy = true;  // train_mp adds up the accuracy of every batch beside its loss
  double sum = 0.0, sum_accuracy = 0.0;
  dlb_status st = DLB_OK;
  gather(mb, 0, 0);
  st = dlb_model_stage_batch(m, rows_of(mb, 0), mb->host_x[0], mb->host_y[0]);
  for (size_t k = 0; k < mb->n_batch && st == DLB_OK; ++k) {
    if (k + 1 < mb->n_batch) {
      // The step that read staging slot (k + 1) % 2 last was step k - 1, whose
      // loss the host has waited for.
      const int slot = (int)((k + 1) & 1);
      gather(mb, k + 1, slot);
      st = dlb_model_stage_batch(m, rows_of(mb, k + 1), mb->host_x[slot], mb->host_y[slot]);
      if (st != DLB_OK) break;
    }
    if (world > 1) st = dlb_model_set_global_batch(m, rows_of(mb, k) * world);
    double batch_loss = 0.0;
    if (st == DLB_OK) st = dlb_model_train_step_staged(m, &batch_loss);
    sum += batch_loss;
    sum_accuracy += m->step_accuracy;
  }
  m->training_size = saved_training;
  m->global_rows = saved_global;
  m->training_accuracy = saved_accuracy;
  if (st != DLB_OK) return st;
  m->hp.epoch_time_step += 1.f;
  *loss = sum / (double)mb->n_batch;
  mb->accuracy = sum_accuracy / (double)mb->n_batch;
  return DLB_OK;
}

// Mean of the batch accuracies of the last dlb_minibatch_train, in percent
// (what train_mp hands to Model::set_accu(ENV::TRAIN, ...)).
double dlb_minibatch_get_accuracy(const dlb_minibatch *mb) { return mb ? mb->accuracy : 0.0; }

}  // extern "C"
