// The host-side Model's state: layers, hyperparameters and device buffers.
// Shared by model.cu (construction and the step) and checkpoint.cu (the
// reference's text checkpoint format).
#pragma once

#include <condition_variable>
#include <functional>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"


// A few host threads that stay around for the row gathers of a model (creating
// threads per call cost more than the gather of a 16 MB batch).  run(parts, fn)
// calls fn(0 .. parts - 1), each once, on the workers and the calling thread,
// and returns when all are done.
class HostWorkers {
 public:
  explicit HostWorkers(size_t threads);
  ~HostWorkers();
  void run(size_t parts, const std::function<void(size_t)> &fn);
  size_t size() const { return threads_.size() + 1; }

 private:
  void loop();
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable work_, done_;
  const std::function<void(size_t)> *fn_ = nullptr;
  size_t parts_ = 0, next_ = 0, finished_ = 0;
  bool stop_ = false;
};

struct LayerRT {
  int type = 0;
  size_t units = 0;
  int af = 0;            // 0 = not set / outside the supported set
  int norm = DLB_NORM_NONE;
  int dropout = DLB_DROPOUT_NONE;
  float dropout_value = 0.f;
  // Indices into the flat parameter vector.
  size_t first_conn = 0, last_conn = 0, first_bias = 0, last_bias = 0, first_norm_unit = 0;
  size_t fan_in = 0;
  // IndRNN layer: its recurrent weights u[units] follow its W inside
  // [first_conn, last_conn) (v1/learner/connections_prepare.cpp L:46-81).
  size_t first_recurrent = 0;
  // Bounds of the recurrent weights when set by hand
  // (Set__Regularization__Constraint_Recurrent_Weight); otherwise the default
  // derived from clip_gradient and seq_w applies.  0 / 0: no clamp.
  bool rec_custom = false;
  float rec_lower = 0.f, rec_upper = 0.f;
  // LSTM layer: `blocks` memory blocks of `cells` cells, units = blocks * cells
  // outputs.  Its products run on packed copies of its weights (lstm.cu): G =
  // units + 3 * blocks rows {z per cell | i | f | o per block}.
  size_t blocks = 0, cells = 0;
  float *lstm_wff = nullptr, *lstm_wrec = nullptr, *lstm_bias = nullptr, *lstm_peep = nullptr;   // [G, I], [G, C], [G], [3, C]
  float *lstm_dwff = nullptr, *lstm_dwrec = nullptr, *lstm_dbias = nullptr, *lstm_dpeep = nullptr;
  unsigned long long *lstm_map_ff = nullptr, *lstm_map_rec = nullptr, *lstm_map_bias = nullptr, *lstm_map_peep = nullptr;
  // Per batch: sums W x_t of all time steps [T, rows, G], R h_{t-1} of one step
  // [rows, G], cell inputs, states, activated states [T, rows, C], gates [T,
  // rows, B], the gates' errors [T, rows, G] and the state errors of two steps.
  float *lstm_gin = nullptr, *lstm_grec = nullptr, *lstm_z = nullptr, *lstm_c = nullptr, *lstm_ca = nullptr;
  float *lstm_gi = nullptr, *lstm_gf = nullptr, *lstm_go = nullptr, *lstm_d = nullptr, *lstm_dc = nullptr;
  // Residual blocks (the reference's layer list: a RESIDUAL layer of depth d
  // followed by its d block layers, v1/learner/compile.cpp).
  int group = 0;            // 1 = layer inside a residual block
  size_t depth = 0;         // RESIDUAL: number of block layers
  size_t pad = 0;           // RESIDUAL: first column of the narrower of shortcut and block in the output
  bool block_input = false; // first layer of a block: no activation in front
  // Owner-computes update across ranks: the reduce-scatter of the layer's
  // weight gradient and the gather of its updated weights are behind these.
  cudaEvent_t ev_reduced = nullptr, ev_gathered = nullptr;
  bool error_final = false; // backward: delta already holds the error w.r.t. Z (the product above formed it)
  size_t norm_units = 0;    // normalised units: width, or fan-in for a block layer
  // Device buffers (allocated by ensure_batch).  Stand-alone FC layer: Z sums,
  // A output after activation and dropout, delta error w.r.t. Z.  Block layer:
  // IN its GEMM input (activation of the previous block layer's sums), A its
  // sums, delta error w.r.t. the sums.  RESIDUAL layer: A = shortcut + block,
  // delta = error of that output.
  float *Z = nullptr, *A = nullptr, *A_lo = nullptr, *delta = nullptr, *delta_lo = nullptr;
  float *IN = nullptr, *IN_lo = nullptr;
  float *stats = nullptr;  // mean | sigma | mean_avg | sigma_avg | r | d, each [T*norm_units]
  uint8_t *mask = nullptr; // [T*units]
  float *uout = nullptr;   // UOut draws of U(-beta, beta), [uout_rows, units (fan-in for a block layer)]
  size_t uout_rows = 0;
  double *fwd_sums = nullptr, *bwd_sums = nullptr;
  // ShakeDrop of a RESIDUAL layer: row flags and the forward / backward draws.
  uint8_t *sd_mask = nullptr;
  float *sd_fwd = nullptr, *sd_bwd = nullptr;
  size_t sd_rows = 0;
};

struct HParams {
  float adam_learning_rate = 0.001f, adam_beta1 = 0.9f, adam_beta2 = 0.999f,
        adam_previous_beta2 = 0.f, adam_epsilon = 1e-8f, adam_gamma = 0.1f,
        learning_rate_final = 0.1f, learning_gamma = 1e-3f, weight_decay = 0.f,
        optimizer_time_step = 0.f, epoch_time_step = 1.f;
  bool use_adam_bias_correction = true;
  bool use_normalized_weight_decay = true;  // model.hpp L:2840
  // Gradient descent (model.hpp L:3020-3022, L:2839).
  float learning_rate = 0.01f, learning_momentum = 0.9f;
  bool use_nesterov = false;
  float regularization_l2 = 0.f;  // kept and saved; without effect on the step, as in the reference
  // Model defaults, v1/learner/model.hpp L:3045-3048.
  float normalization_momentum_average = 0.999f, normalization_epsilon = 1e-5f,
        brn_r_max = 1.f, brn_d_max = 0.f;
};


struct dlb_model {
  dlb_ctx *ctx = nullptr;
  std::vector<LayerRT> layers;
  size_t seq_w = 1, n_time_delay = 0;
  int model_type = DLB_MODEL_FEEDFORWARD;
  int loss = 0, optimizer = 0;
  HParams hp;
  size_t total_weights = 0, total_bias = 0, total_norm_units = 0, total_parameters = 0;
  bool any_norm = false;
  size_t max_batch = 0, alloc_rows = 0, global_rows = 0;
  size_t training_size = 0;  // examples of the training set; 0: one batch is the whole set
  unsigned weight_seed = 5489u;
  std::mt19937 weight_gen;
  // Flat device vectors.
  float *params = nullptr, *params_lo = nullptr, *grads = nullptr, *m1 = nullptr, *m2 = nullptr,
        *m2hat = nullptr;
  float *input = nullptr, *input_lo = nullptr, *target = nullptr;
  // Time-stepped models: the caller's rows [rows, T*n] as they arrive, before
  // the reorder to [T, rows, n].
  float *input_rows = nullptr, *target_rows = nullptr;
  float *wd_mask = nullptr;  // [P]: 1 where weight decay applies
  // Model::use_clip_gradient / clip_gradient (model.hpp defaults: off, 1).
  bool use_clip_gradient = false;
  float clip_gradient = 1.f;
  // Evaluation (Driver::evalt): propagation state, accuracy function and its
  // counter; r = 1 and d = 0 for the normalization by running averages.
  int propagation = DLB_PROPAGATION_TRAINING;
  int accu_fn = DLB_ACCU_DISTANCE;   // v1/learner/model.hpp L:157
  float accu_var = 0.49f;            // L:3019
  double *accu_sum = nullptr;
  bool training_accuracy = false;    // compute_error counts the accuracy too (one more pass over the outputs)
  float *ones = nullptr, *zeros = nullptr;
  size_t const_units = 0;
  float *stage_x = nullptr, *stage_y = nullptr;  // pinned
  size_t stage_x_elems = 0, stage_y_elems = 0;
  // Row-pointer inputs (forward_pass / compute_error / compute_loss) cross on the
  // copy stream: [0] inputs, [1] targets.  copied: the copy out of the staging
  // buffer is done (the host may refill it); consumed: the kernels that read
  // the device tensor have been enqueued up to here (the next copy waits).
  cudaEvent_t rows_copied[2] = {nullptr, nullptr}, rows_consumed[2] = {nullptr, nullptr};
  bool rows_in_flight[2] = {false, false};
  // Batches copied ahead of the step that uses them: two device slots filled
  // on a stream of their own, so that the copy of batch i+1 runs under the
  // kernels of batch i.
  struct Ahead {
    float *x = nullptr, *y = nullptr;
    size_t x_elems = 0, y_elems = 0, rows = 0;
    cudaEvent_t ready = nullptr, consumed = nullptr;
    bool in_use = false;  // `consumed` has been recorded at least once
  } ahead[2];
  cudaStream_t copy_stream = nullptr;
  HostWorkers *workers = nullptr;   // row gathers of forward_pass / compute_error / compute_loss
  size_t ahead_head = 0, ahead_tail = 0;  // staged so far, consumed so far
  double *loss_sum = nullptr;
  // The loss of a one-call step leaves the device asynchronously: a device copy of the
  // sum, its exchange across ranks, a copy into page-locked host memory and an
  // event, two slots used in turn, so that the update is enqueued before the
  // host waits.  loss_lag = 1: a staged step returns the loss of the step before.
  double *loss_tmp = nullptr;       // device [2 slots][loss sum, accuracy counter]
  double *loss_host = nullptr;      // page-locked, the same
  double step_accuracy = 0.0;       // percent, of the step whose loss was collected last
  cudaEvent_t loss_ready[2] = {nullptr, nullptr};
  size_t loss_rows_at[2] = {0, 0};
  bool loss_valid[2] = {false, false};
  size_t loss_steps = 0;
  int loss_lag = 0;
  size_t loss_rows = 0;  // rows accumulated since reset_loss
  bool params_lo_valid = false;
  uint64_t plane_generation = 0;  // the context's value when the weights were last split
  // Inside train_step the step is known to be a single chunk, so each layer's
  // weight gradient is all-reduced as soon as its GEMM has been enqueued.
  bool overlap_grad_allreduce = false;
  // The gradient vector is all zero (fresh, or cleared by the last update), so
  // the weight-gradient products may overwrite instead of accumulate.
  bool grads_clean = false;
  // Multi-GPU one-call steps of plain stacks: each rank updates the rows of
  // every weight matrix it owns (reduce-scatter of the gradient, update of
  // the slice, gather of the weights) instead of all ranks updating all of it.
  // moments_sharded: the moments of the weight matrices are current only on
  // their owners' slices.  update_prepared: the step's scalars were drawn
  // during the backward pass and the weight matrices are already updated.
  bool sharded_update = true;
  bool moments_sharded = false;
  bool update_prepared = false;
  dlb_optimizer_scalars update_k = {};
};
