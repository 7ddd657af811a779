// Host-side Model: the reference's v1::Model construction, parameter layout and
// step entry points (lib/deep-learning/v1/learner/model.hpp L:752-3384), with
// every tensor resident in HBM and every numerical step dispatched to the
// kernels of this library through its C ABI.  No arithmetic of the step runs on
// the host.
//
// Device memory per model:
//   params, grads, first/second(/hat) moments, and the TF32 residual plane of
//   the weight block: flat [P] (the reference's ptr_array_parameters order);
//   per layer and time step: Z (pre-normalisation sums), A (output, after
//   dropout), A_lo, delta (error w.r.t. Z), delta_lo, all [rows, units];
//   per normalised layer: mean, sigma, running averages, r, d [T, units];
//   double sums for the statistics exchanges.
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <atomic>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"
#include "model.cuh"

using namespace dlb;

namespace {

size_t n_in(const dlb_model *m) { return m->layers.front().units; }
size_t n_out(const dlb_model *m) { return m->layers.back().units; }

// Plain batch normalization (Forward_Pass__Batch_Normalization__Training__OpenMP,
// fwp_mp.cpp L:4493-4603, backward bwp_mp.cpp L:1265-1385) is batch
// renormalization with r = 1 and d = 0, which the clips give with these bounds.
float r_max_of(const dlb_model *m, const LayerRT &l) {
  return l.norm == DLB_NORM_BATCH_NORMALIZATION ? 1.f : m->hp.brn_r_max;
}
float d_max_of(const dlb_model *m, const LayerRT &l) {
  return l.norm == DLB_NORM_BATCH_NORMALIZATION ? 0.f : m->hp.brn_d_max;
}

// mag of the IndRNN bounds: clip(clip_gradient, 2, 10)
// (v1/ops/constraints/constraint.cpp L:66, v1/learner/model.cpp L:5303, L:5336).
float indrnn_magnitude(const dlb_model *m) { return fminf(fmaxf(m->clip_gradient, 2.f), 10.f); }

bool is_indrnn(const LayerRT &l) { return l.type == DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT; }
bool is_lstm(const LayerRT &l) { return l.type == DLB_LAYER_LSTM; }
// Layer i holds the error of a softmax output: its columns are the classes,
// and the classes nobody is wrong about have errors many orders of magnitude
// below the others' once the model has learnt something, so the layer's weight
// gradient takes planes with a scale per class.
bool class_error(const dlb_model *m, size_t i) {
  return i + 1 == m->layers.size() && m->layers[i].af == DLB_AF_SOFTMAX;
}
size_t lstm_gates(const LayerRT &l) { return l.units + 3 * l.blocks; }

// Bounds the recurrent weights of an IndRNN layer are clamped to after an
// update: the ones set by hand, else +-mag^(1/T) with mag = clip(clip_gradient,
// 2, 10) = 2 with the reference's default clip_gradient of 1; every activation of
// the supported set is in a class that takes this default
// (Compute__Regularization__Constraint_Recurrent_Weight__Default,
// v1/ops/constraints/constraint.cpp L:64-95).
void recurrent_bounds(const dlb_model *m, const LayerRT &l, float *lo, float *hi) {
  if (l.rec_custom) {
    *lo = l.rec_lower;
    *hi = l.rec_upper;
    return;
  }
  const float bound = powf(indrnn_magnitude(m), 1.f / (float)m->seq_w);
  *lo = -bound;
  *hi = bound;
}

// Models that run the [T, rows, n] path: more than one time step, or an IndRNN
// layer (whose recurrence is then empty at T = 1).
bool time_stepped(const dlb_model *m) {
  if (m->seq_w > 1) return true;
  for (const LayerRT &l : m->layers)
    if (is_indrnn(l) || is_lstm(l)) return true;
  return false;
}

dlb_status dev_alloc(dlb_model *m, float **p, size_t elems, bool zero) {
  if (*p) {
    DLB_TRY(dlb_free(m->ctx, *p));
    *p = nullptr;
  }
  DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(p), elems * sizeof(float)));
  if (zero) DLB_TRY(dlb_memset(m->ctx, *p, 0, elems * sizeof(float)));
  return DLB_OK;
}

// Parameter layout { W per layer | bias per layer | gamma per unit | beta per
// unit }; gamma/beta exist for every unit of every layer as soon as one layer
// is normalised (compile.cpp L:610-695, allocate.cpp L:1150-1176).
dlb_status layout_parameters(dlb_model *m) {
  // Graph: fan-in of every FC layer, width of every RESIDUAL layer (that of the
  // layer below it), and the number of normalised units (a block layer
  // normalises its input, so it has fan-in many).
  size_t width = m->layers[0].units;
  m->layers[0].norm_units = width;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) {
      DLB_REQUIRE(l.depth >= 1 && i + l.depth < m->layers.size(),
                  "compile: a RESIDUAL layer needs its block layers and a layer after them");
      l.group = 0;
      size_t fan = width;
      for (size_t j = 1; j <= l.depth; ++j) {
        LayerRT &b = m->layers[i + j];
        DLB_REQUIRE(b.type == DLB_LAYER_FULLY_CONNECTED, "compile: block layers must be fully connected");
        b.group = 1;
        b.block_input = j == 1;
        b.fan_in = fan;
        b.norm_units = fan;
        fan = b.units;
      }
      // As wide as the wider of shortcut and block; the narrower one enters
      // from column pad on; the layer's own normalization acts on the block
      // output (v1/learner/compile.cpp L:337-352).
      l.units = std::max(width, fan);
      l.pad = ((width > fan ? width - fan : fan - width) + 1) / 2;
      l.norm_units = fan;
      l.fan_in = width;  // width of the shortcut
      width = l.units;
      i += l.depth;
    } else {
      l.group = 0;
      l.block_input = false;
      l.fan_in = width;
      l.norm_units = l.units;
      width = l.units;
    }
  }
  size_t w = 0;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;
    l.first_conn = w;
    if (is_lstm(l)) {
      // Per block: per cell [W_z | R_z], W_i W_f W_o, R_i R_f R_o, p_i p_f p_o
      // (Prepare__Connections__LSTM, v1/learner/connections_prepare.cpp L:83-225).
      w += l.blocks * (l.cells * (l.fan_in + l.units) + 3 * l.fan_in + 3 * l.units + 3 * l.cells);
      l.last_conn = w;
      continue;
    }
    w += l.units * l.fan_in;
    if (l.type == DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT) {
      l.first_recurrent = w;
      w += l.units;
    }
    l.last_conn = w;
  }
  m->total_weights = w;
  size_t b = w;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;
    l.first_bias = b;
    b += is_lstm(l) ? lstm_gates(l) : l.units;  // Prepare__Bias__LSTM: cells, then three per block
    l.last_bias = b;
  }
  m->total_bias = b - w;
  m->any_norm = false;
  for (auto &l : m->layers) m->any_norm |= l.norm != DLB_NORM_NONE;
  size_t u = 0;
  for (auto &l : m->layers) {
    l.first_norm_unit = u;
    u += l.norm_units;
  }
  m->total_norm_units = m->any_norm ? u : 0;
  m->total_parameters = m->total_weights + m->total_bias + 2 * m->total_norm_units;
  return DLB_OK;
}

size_t gamma_index(const dlb_model *m, const LayerRT &l) {
  return m->total_weights + m->total_bias + l.first_norm_unit;
}
size_t beta_index(const dlb_model *m, const LayerRT &l) {
  return m->total_weights + m->total_bias + m->total_norm_units + l.first_norm_unit;
}

// (Re)allocates the flat vectors, keeping existing weights and biases when the
// normalisation block is added later, as the reference's reallocation does.
// Packed weight buffers of the LSTM layers and the maps from their rows to the
// flat parameter vector (offsets in floats), for gather before the forward pass
// and scatter-add of the gradients.  Bias offsets are the reference's own: its
// kernels index the layer's biases from first_bias_connection_index, which
// Prepare__Bias__LSTM leaves at the block part (connections_prepare.cpp
// L:240-262), so b_z[c] sits units entries into the layer's reserved range, the
// gates behind it, the last `units` of them in the next layer's biases.
dlb_status lstm_prepare(dlb_model *m) {
  for (size_t li = 1; li < m->layers.size(); ++li) {
    LayerRT &l = m->layers[li];
    if (!is_lstm(l)) continue;
    const size_t I = l.fan_in, C = l.units, B = l.blocks, K = l.cells, G = lstm_gates(l);
    std::vector<unsigned long long> ff(G), rec(G), bias(G), peep(3 * C);
    size_t w = l.first_conn;
    for (size_t b = 0; b < B; ++b) {
      for (size_t k = 0; k < K; ++k) {
        ff[b * K + k] = w;
        w += I;
        rec[b * K + k] = w;
        w += C;
      }
      for (size_t g = 0; g < 3; ++g) {
        ff[C + g * B + b] = w;
        w += I;
      }
      for (size_t g = 0; g < 3; ++g) {
        rec[C + g * B + b] = w;
        w += C;
      }
      for (size_t g = 0; g < 3; ++g)
        for (size_t k = 0; k < K; ++k) peep[g * C + b * K + k] = w++;
    }
    DLB_REQUIRE(w == l.last_conn, "lstm: parameter layout");
    const size_t base = l.first_bias + C;
    DLB_REQUIRE(base + G <= m->total_parameters,
                "lstm: the layer after an LSTM layer must have at least as many units as the LSTM layer has cells "
                "(the reference's bias indices reach that far past the layer's own biases)");
    for (size_t g = 0; g < G; ++g) bias[g] = base + g;
    struct { unsigned long long **dev; std::vector<unsigned long long> *host; } maps[] = {
        {&l.lstm_map_ff, &ff}, {&l.lstm_map_rec, &rec}, {&l.lstm_map_bias, &bias}, {&l.lstm_map_peep, &peep}};
    for (auto &mp : maps) {
      if (*mp.dev) DLB_TRY(dlb_free(m->ctx, *mp.dev));
      *mp.dev = nullptr;
      DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(mp.dev), mp.host->size() * sizeof(unsigned long long)));
      DLB_TRY(dlb_memcpy_h2d(m->ctx, *mp.dev, mp.host->data(), mp.host->size() * sizeof(unsigned long long)));
    }
    DLB_TRY(dlb_ctx_sync(m->ctx, nullptr));  // the host vectors go out of scope
    DLB_TRY(dev_alloc(m, &l.lstm_wff, G * I, false));
    DLB_TRY(dev_alloc(m, &l.lstm_wrec, G * C, false));
    DLB_TRY(dev_alloc(m, &l.lstm_bias, G, false));
    DLB_TRY(dev_alloc(m, &l.lstm_peep, 3 * C, false));
    DLB_TRY(dev_alloc(m, &l.lstm_dwff, G * I, false));
    DLB_TRY(dev_alloc(m, &l.lstm_dwrec, G * C, true));
    DLB_TRY(dev_alloc(m, &l.lstm_dbias, G, false));
    DLB_TRY(dev_alloc(m, &l.lstm_dpeep, 3 * C, false));
  }
  return DLB_OK;
}

dlb_status allocate_parameters(dlb_model *m) {
  const size_t old_wb = m->params ? m->total_weights + m->total_bias : 0;
  std::vector<float> keep;
  if (m->params && old_wb) {
    keep.resize(old_wb);
    DLB_TRY(dlb_memcpy_d2h(m->ctx, keep.data(), m->params, old_wb * sizeof(float)));
  }
  DLB_TRY(layout_parameters(m));
  const size_t P = m->total_parameters;
  std::vector<float> host(P, 0.f);
  if (!keep.empty()) memcpy(host.data(), keep.data(), keep.size() * sizeof(float));
  // gamma = 1 (0.1 for an IndRNN layer), beta = 0 (allocate.cpp L:1485-1507).
  if (m->total_norm_units)
    for (const LayerRT &l : m->layers)
      for (size_t i = 0; i < l.norm_units; ++i)
        host[gamma_index(m, l) + i] =
            l.type == DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT ? 0.1f : 1.f;
  DLB_TRY(dev_alloc(m, &m->params, P, false));
  DLB_TRY(dlb_memcpy_h2d(m->ctx, m->params, host.data(), P * sizeof(float)));
  DLB_TRY(dlb_ctx_sync(m->ctx, nullptr));
  DLB_TRY(dev_alloc(m, &m->params_lo, m->total_weights ? m->total_weights : 4, true));
  DLB_TRY(dev_alloc(m, &m->grads, P, true));
  DLB_TRY(dev_alloc(m, &m->m1, P, true));
  DLB_TRY(dev_alloc(m, &m->m2, P, true));
  DLB_TRY(dev_alloc(m, &m->m2hat, P, true));
  if (m->wd_mask) {
    DLB_TRY(dlb_free(m->ctx, m->wd_mask));
    m->wd_mask = nullptr;
  }
  DLB_TRY(lstm_prepare(m));
  m->grads_clean = true;
  m->params_lo_valid = false;
  return DLB_OK;
}

dlb_status free_batch_buffers(dlb_model *m) {
  for (auto &l : m->layers) {
    float **bufs[] = {&l.Z, &l.A, &l.A_lo, &l.delta, &l.delta_lo, &l.IN, &l.IN_lo, &l.lstm_gin, &l.lstm_grec,
                      &l.lstm_z, &l.lstm_c, &l.lstm_ca, &l.lstm_gi, &l.lstm_gf, &l.lstm_go, &l.lstm_d, &l.lstm_dc};
    planes_rows_exempt(m->ctx, l.delta_lo, 0, false);
    for (float **b : bufs) {
      if (*b) DLB_TRY(dlb_free(m->ctx, *b));
      *b = nullptr;
    }
  }
  float **bufs[] = {&m->input, &m->input_lo, &m->target, &m->input_rows, &m->target_rows};
  for (float **b : bufs) {
    if (*b) DLB_TRY(dlb_free(m->ctx, *b));
    *b = nullptr;
  }
  m->alloc_rows = 0;
  return DLB_OK;
}

dlb_status ensure_norm_state(dlb_model *m) {
  const size_t T = m->seq_w;
  for (auto &l : m->layers) {
    if (l.norm == DLB_NORM_NONE || l.stats) continue;
    const size_t n = T * l.norm_units;
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.stats), 6 * n * sizeof(float)));
    std::vector<float> h(6 * n, 0.f);
    for (size_t i = 0; i < n; ++i) h[3 * n + i] = 1.f;  // running sigma = 1 (allocate.cpp L:1281-1284)
    DLB_TRY(dlb_memcpy_h2d(m->ctx, l.stats, h.data(), h.size() * sizeof(float)));
    DLB_TRY(dlb_ctx_sync(m->ctx, nullptr));
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.fwd_sums), 2 * n * sizeof(double)));
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.bwd_sums), 5 * n * sizeof(double)));
  }
  // An IndRNN layer without normalization still needs the per-step du sums.
  for (auto &l : m->layers) {
    if (l.type != DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT || l.bwd_sums) continue;
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.bwd_sums), T * l.units * sizeof(double)));
  }
  return DLB_OK;
}

dlb_status ensure_masks(dlb_model *m) {
  for (auto &l : m->layers) {
    const bool bern = l.dropout == DLB_DROPOUT_BERNOULLI || l.dropout == DLB_DROPOUT_BERNOULLI_INVERTED;
    if (!bern || l.mask) continue;
    const size_t n = m->seq_w * l.units;
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.mask), n));
    DLB_TRY(dlb_memset(m->ctx, l.mask, 1, n));  // keep everything until a mask is set
  }
  return DLB_OK;
}

// Activation / error buffers for `rows` rows (the reference's
// update_mem_batch_size, v1/learner/update_size.cpp L:169-205).
dlb_status ensure_batch(dlb_model *m, size_t rows) {
  if (!m->params) DLB_TRY(allocate_parameters(m));
  DLB_TRY(ensure_norm_state(m));
  DLB_TRY(ensure_masks(m));
  if (rows <= m->alloc_rows) return DLB_OK;
  DLB_TRY(free_batch_buffers(m));
  const size_t T = m->seq_w;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    const size_t n = T * rows * l.units;
    DLB_TRY(dev_alloc(m, &l.A, n, false));
    DLB_TRY(dev_alloc(m, &l.delta, n, false));
    if (l.type == DLB_LAYER_RESIDUAL) {
      DLB_TRY(dev_alloc(m, &l.A_lo, n, false));
      continue;
    }
    DLB_TRY(dev_alloc(m, &l.delta_lo, n, false));
    // Errors of the backward pass, one row per example (and time step).
    planes_rows_exempt(m->ctx, l.delta_lo, n * sizeof(float), true);
    if (is_lstm(l)) {
      const size_t TB = T * rows, G = lstm_gates(l);
      DLB_TRY(dev_alloc(m, &l.A_lo, n, false));
      DLB_TRY(dev_alloc(m, &l.lstm_gin, TB * G, false));
      DLB_TRY(dev_alloc(m, &l.lstm_grec, rows * G, false));
      DLB_TRY(dev_alloc(m, &l.lstm_z, n, false));
      DLB_TRY(dev_alloc(m, &l.lstm_c, n, false));
      DLB_TRY(dev_alloc(m, &l.lstm_ca, n, false));
      DLB_TRY(dev_alloc(m, &l.lstm_gi, TB * l.blocks, false));
      DLB_TRY(dev_alloc(m, &l.lstm_gf, TB * l.blocks, false));
      DLB_TRY(dev_alloc(m, &l.lstm_go, TB * l.blocks, false));
      DLB_TRY(dev_alloc(m, &l.lstm_d, TB * G, false));
      DLB_TRY(dev_alloc(m, &l.lstm_dc, 2 * rows * l.units, false));
      continue;
    }
    if (l.group == 1) {
      // Block layer: A holds its sums; later layers also keep their GEMM input.
      if (!l.block_input) {
        DLB_TRY(dev_alloc(m, &l.IN, T * rows * l.fan_in, false));
        DLB_TRY(dev_alloc(m, &l.IN_lo, T * rows * l.fan_in, false));
      }
    } else {
      DLB_TRY(dev_alloc(m, &l.Z, n, false));
      DLB_TRY(dev_alloc(m, &l.A_lo, n, false));
    }
  }
  DLB_TRY(dev_alloc(m, &m->input, T * rows * n_in(m), false));
  DLB_TRY(dev_alloc(m, &m->input_lo, T * rows * n_in(m), false));
  DLB_TRY(dev_alloc(m, &m->target, T * rows * n_out(m), false));
  if (time_stepped(m)) {
    DLB_TRY(dev_alloc(m, &m->input_rows, T * rows * n_in(m), false));
    DLB_TRY(dev_alloc(m, &m->target_rows, T * rows * n_out(m), false));
  }
  if (!m->loss_sum) {
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&m->loss_sum), sizeof(double)));
    DLB_TRY(dlb_memset(m->ctx, m->loss_sum, 0, sizeof(double)));
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&m->accu_sum), sizeof(double)));
    DLB_TRY(dlb_memset(m->ctx, m->accu_sum, 0, sizeof(double)));
  }
  m->alloc_rows = rows;
  return DLB_OK;
}

dlb_brn_unit_arrays unit_arrays(dlb_model *m, LayerRT &l, size_t t) {
  const size_t n = m->seq_w * l.norm_units;
  dlb_brn_unit_arrays u;
  float *s = l.stats + t * l.norm_units;
  u.mean = s;
  u.sigma = s + n;
  u.mean_average = s + 2 * n;
  u.sigma_average = s + 3 * n;
  u.r = s + 4 * n;
  u.d = s + 5 * n;
  u.gamma = m->params + gamma_index(m, l);
  u.beta = m->params + beta_index(m, l);
  return u;
}

bool af_supported(int af) {
  switch (af) {
    case DLB_AF_ELU: case DLB_AF_ISRLU: case DLB_AF_LINEAR: case DLB_AF_LEAKY_RELU:
    case DLB_AF_RELU: case DLB_AF_SELU: case DLB_AF_SOFTMAX: return true;
    default: return false;
  }
}

dlb_status check_supported(dlb_model *m) {
  if (m->layers.size() < 2) {
    set_error("model: compile() has not been called");
    return DLB_ERR_INVALID;
  }
  if (m->model_type != DLB_MODEL_FEEDFORWARD && m->model_type != DLB_MODEL_RECURRENT) {
    set_error("model: model type %d is outside the supported path (FEEDFORWARD, RECURRENT)", m->model_type);
    return DLB_ERR_UNSUPPORTED;
  }
  if (m->seq_w > 1 && m->model_type != DLB_MODEL_RECURRENT) {
    set_error("model: seq_w %zu needs model type RECURRENT", m->seq_w);
    return DLB_ERR_INVALID;
  }
  const bool stepped = time_stepped(m);
  for (size_t i = 1; i < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    if (stepped) {
      // The time-stepped path covers stacks of IndRNN and fully connected
      // layers with batch renormalization between them and Bernoulli dropout
      // (plain or inverted) on their outputs.
      // Residual blocks of fully connected layers run too (ShakeDrop on the
      // block, Bernoulli dropout inside it).
      const bool bern = l.dropout == DLB_DROPOUT_BERNOULLI || l.dropout == DLB_DROPOUT_BERNOULLI_INVERTED;
      const bool shake = l.type == DLB_LAYER_RESIDUAL && l.dropout == DLB_DROPOUT_SHAKEDROP;
      const bool uout = l.dropout == DLB_DROPOUT_UOUT && l.group == 0 && l.type != DLB_LAYER_RESIDUAL;
      if (l.dropout != DLB_DROPOUT_NONE && !bern && !shake && !uout) {
        set_error("model: layer %zu: dropout other than Bernoulli, UOut on a layer outside a block and ShakeDrop "
                  "on a residual layer is outside the supported path of time-stepped (recurrent) models", i);
        return DLB_ERR_UNSUPPORTED;
      }
      if (l.group == 1 && is_indrnn(l)) {
        set_error("model: layer %zu: recurrent layers inside a residual block are outside the supported path", i);
        return DLB_ERR_UNSUPPORTED;
      }
      if (is_indrnn(l) && (i + 1 == m->layers.size() || l.af == DLB_AF_SOFTMAX)) {
        set_error("model: layer %zu: an IndRNN layer is a hidden layer with an element-wise activation", i);
        return DLB_ERR_UNSUPPORTED;
      }
    }
    if (is_indrnn(l)) {
      if (!af_supported(l.af)) {
        set_error("model: layer %zu activation %d is outside the supported set", i, l.af);
        return DLB_ERR_UNSUPPORTED;
      }
      continue;
    }
    if (is_lstm(l)) {
      // Unidirectional, tanh / sigmoid as the reference fixes them
      // (connections_prepare.cpp L:123-124), peepholes; no normalization, dropout
      // or zoneout on the layer, not inside a residual block.
      if (l.norm != DLB_NORM_NONE || l.dropout != DLB_DROPOUT_NONE || l.group == 1 || i + 1 == m->layers.size()) {
        set_error("model: LSTM layer %zu: normalization, dropout, a place inside a residual block or as output "
                  "layer are outside the supported path", i);
        return DLB_ERR_UNSUPPORTED;
      }
      continue;
    }
    if (l.type == DLB_LAYER_RESIDUAL) {
      if (m->layers[i + 1].norm != DLB_NORM_NONE) {
        set_error("model: normalization on the first layer of a residual block (layer %zu) is outside "
                  "the supported path", i + 1);
        return DLB_ERR_UNSUPPORTED;
      }
      continue;
    }
    if (l.type != DLB_LAYER_FULLY_CONNECTED) {
      set_error("model: layer %zu has type %d; only fully connected and residual layers are supported",
                i, l.type);
      return DLB_ERR_UNSUPPORTED;
    }
    if (l.block_input) continue;  // its activation is never applied (fwp_mp.cpp L:4003)
    if (!af_supported(l.af)) {
      set_error("model: layer %zu activation %d is outside the supported set "
                "(the reference's default for a fully connected layer is SIGMOID; set one of "
                "RELU/LEAKY_RELU/ELU/SELU/ISRLU/LINEAR/SOFTMAX)", i, l.af);
      return DLB_ERR_UNSUPPORTED;
    }
    if (l.af == DLB_AF_SOFTMAX && i + 1 != m->layers.size()) {
      set_error("model: softmax is only supported on the output layer");
      return DLB_ERR_UNSUPPORTED;
    }
  }
  return DLB_OK;
}

dlb_status refresh_weight_residuals(dlb_model *m) {
  // A change of the context's operand form since the last split makes the
  // weight planes stale.
  if (m->plane_generation != m->ctx->plane_generation) {
    m->plane_generation = m->ctx->plane_generation;
    m->params_lo_valid = false;
  }
  if (m->params_lo_valid || m->total_weights == 0) return DLB_OK;
  // One plane buffer per layer, so that every weight matrix gets a scale of its own.
  for (size_t i = 1; i < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;
    DLB_TRY(dlb_split_planes_2d(m->ctx, m->params + l.first_conn, m->params_lo + l.first_conn, (int)l.units,
                                (int)l.fan_in));
  }
  m->params_lo_valid = true;
  return DLB_OK;
}

dlb_status ensure_constants(dlb_model *m, size_t units);

// Normalization by the running averages, the inference form of batch
// normalization and renormalization alike
// (Forward_Pass__Batch_Normalization__Inference__OpenMP, fwp_mp.cpp
// L:4461-4491): gamma (z - running mean) / running sigma + beta, i.e. the
// training formula with r = 1 and d = 0.  Covers all time steps of the layer.
dlb_status inference_arrays(dlb_model *m, LayerRT &l, dlb_brn_unit_arrays *u) {
  DLB_TRY(ensure_constants(m, m->seq_w * l.norm_units));
  *u = unit_arrays(m, l, 0);
  u->mean = u->mean_average;
  u->sigma = u->sigma_average;
  u->r = m->ones;
  u->d = m->zeros;
  return DLB_OK;
}

// Batch-renormalization statistics of layer l over `in` [B, l.norm_units]:
// sums, exchange across ranks, averages and corrections; the running averages
// alone in an inference pass.
dlb_status norm_statistics(dlb_model *m, LayerRT &l, const float *in, int B, dlb_brn_unit_arrays *u) {
  if (m->propagation == DLB_PROPAGATION_INFERENCE) return inference_arrays(m, l, u);
  const int Bg = (int)(m->global_rows ? m->global_rows : (size_t)B);
  const int n = (int)l.norm_units;
  *u = unit_arrays(m, l, 0);
  DLB_TRY(dlb_brn_forward_sums(m->ctx, in, B, n, l.fwd_sums));
  DLB_TRY(dlb_allreduce_f64(m->ctx, l.fwd_sums, 2 * (size_t)n));
  return dlb_brn_forward_finalize(m->ctx, l.fwd_sums, Bg, n, m->hp.normalization_momentum_average,
                                  m->hp.normalization_epsilon, r_max_of(m, l), d_max_of(m, l), u);
}

// Backward of the same: the four sums, d_gamma / d_beta into the gradient
// vector, exchange of d_mean / d_sigma, and the apply pass.  `e` holds
// delta_af on entry and the error w.r.t. the normalisation input on return.
dlb_status norm_backward(dlb_model *m, LayerRT &l, float *e, float *e_lo, const float *in,
                         const float *act, int af, int B) {
  const int Bg = (int)(m->global_rows ? m->global_rows : (size_t)B);
  const int n = (int)l.norm_units;
  dlb_brn_unit_arrays u = unit_arrays(m, l, 0);
  DLB_TRY(dlb_activation_backward(m->ctx, e, in, act, &u, af, B, n, l.bwd_sums));
  DLB_TRY(dlb_brn_backward_param_grads(m->ctx, l.bwd_sums, n, m->grads + gamma_index(m, l),
                                       m->grads + beta_index(m, l), 1));
  DLB_TRY(dlb_allreduce_f64(m->ctx, l.bwd_sums + 2 * (size_t)n, 2 * (size_t)n));
  return dlb_brn_backward_apply(m->ctx, e, e_lo, in, &u, l.bwd_sums, Bg, B, n);
}

// Arrays of ones and zeros, the r and d of a normalization by running averages.
dlb_status ensure_constants(dlb_model *m, size_t units) {
  if (units <= m->const_units) return DLB_OK;
  if (m->ones) DLB_TRY(dlb_free(m->ctx, m->ones));
  if (m->zeros) DLB_TRY(dlb_free(m->ctx, m->zeros));
  m->ones = m->zeros = nullptr;
  std::vector<float> one(units, 1.f);
  DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&m->ones), units * sizeof(float)));
  DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&m->zeros), units * sizeof(float)));
  DLB_TRY(dlb_memcpy_h2d(m->ctx, m->ones, one.data(), units * sizeof(float)));
  DLB_TRY(dlb_memset(m->ctx, m->zeros, 0, units * sizeof(float)));
  DLB_TRY(dlb_ctx_sync(m->ctx, nullptr));
  m->const_units = units;
  return DLB_OK;
}

// A layer with UOut needs this step's draws for at least B rows.
dlb_status uout_ready(dlb_model *m, const LayerRT &l, size_t index, int B) {
  (void)m;
  if (l.dropout != DLB_DROPOUT_UOUT) return DLB_OK;
  if (!l.uout || l.uout_rows < (size_t)B) {
    set_error("model: layer %zu uses UOut but no noise was set for %d rows (dlb_model_set_uout_noise)",
              index, B);
    return DLB_ERR_INVALID;
  }
  return DLB_OK;
}

// ref: Forward_Pass__Residual__OpenMP and Forward_Pass__Residual__FC__OpenMP
// (v1/learner/fwp_mp.cpp L:3777-3911, L:3951-4192): pre-activation block layers,
// then the residual layer's normalization, ShakeDrop and the shortcut sum.
dlb_status forward_residual(dlb_model *m, size_t i, const float *X, const float *X_lo, int B) {
  LayerRT &res = m->layers[i];
  const bool inference = m->propagation == DLB_PROPAGATION_INFERENCE;
  const float *in = X, *in_lo = X_lo;
  const float *prev_sums = nullptr;
  for (size_t j = 1; j <= res.depth; ++j) {
    LayerRT &b = m->layers[i + j];
    const bool norm = b.norm != DLB_NORM_NONE;
    if (!b.block_input) {
      dlb_brn_unit_arrays u;
      if (norm) DLB_TRY(norm_statistics(m, b, prev_sums, B, &u));
      if (inference) {
        // Plain Bernoulli dropout scales by the keep probability (fwp_mp.cpp L:4870-4892).
        dlb_dropout_desc dp{DROPOUT_INFERENCE_SCALE, b.dropout_value, nullptr, nullptr};
        DLB_TRY(dlb_activation_forward(m->ctx, prev_sums, norm ? &u : nullptr, b.af,
                                       b.dropout == DLB_DROPOUT_BERNOULLI ? &dp : nullptr, b.IN, b.IN_lo, B,
                                       (int)b.fan_in));
      } else {
        DLB_TRY(uout_ready(m, b, i + j, B));
        dlb_dropout_desc dp{b.dropout, b.dropout_value, b.mask, b.uout};
        DLB_TRY(dlb_activation_forward(m->ctx, prev_sums, norm ? &u : nullptr, b.af,
                                       b.dropout != DLB_DROPOUT_NONE ? &dp : nullptr, b.IN, b.IN_lo, B,
                                       (int)b.fan_in));
      }
      in = b.IN;
      in_lo = b.IN_lo;
    }
    const float *bias = norm ? nullptr : m->params + b.first_bias;
    DLB_TRY(dlb_fc_forward(m->ctx, in, in_lo, m->params + b.first_conn, m->params_lo + b.first_conn,
                           bias, b.A, B, (int)b.fan_in, (int)b.units));
    prev_sums = b.A;
  }
  LayerRT &last = m->layers[i + res.depth];
  float *block = last.A;
  // At inference the block output of a ShakeDrop layer is scaled by 1 - p, p the
  // layer's dropout value (fwp_mp.cpp L:3876-3897), in the same pass as the
  // layer's own normalization where it has one.
  dlb_dropout_desc keep{DROPOUT_INFERENCE_SCALE, 1.f - res.dropout_value, nullptr, nullptr};
  const bool scale = inference && res.dropout == DLB_DROPOUT_SHAKEDROP;
  if (res.norm != DLB_NORM_NONE || scale) {
    // The residual layer's own normalization writes to its error buffer's
    // sibling: reuse last.delta as the normalised block output until backward.
    dlb_brn_unit_arrays u;
    if (res.norm != DLB_NORM_NONE) DLB_TRY(norm_statistics(m, res, last.A, B, &u));
    DLB_TRY(dlb_activation_forward(m->ctx, last.A, res.norm != DLB_NORM_NONE ? &u : nullptr, DLB_AF_LINEAR,
                                   scale ? &keep : nullptr, last.delta, nullptr, B, (int)res.units));
    block = last.delta;
  }
  const bool shake = !inference && res.dropout == DLB_DROPOUT_SHAKEDROP;
  if (shake && (!res.sd_mask || res.sd_rows < (size_t)B)) {
    set_error("model: residual layer %zu uses ShakeDrop but no noise was set for %d rows "
              "(dlb_model_set_shakedrop_noise)", i, B);
    return DLB_ERR_INVALID;
  }
  if (last.units != res.fan_in)
    return dlb_residual_forward_padded(m->ctx, X, (int)res.fan_in, block, (int)last.units,
                                       shake ? res.sd_mask : nullptr, shake ? res.sd_fwd : nullptr, res.A,
                                       res.A_lo, B);
  return dlb_residual_forward(m->ctx, X, block, shake ? res.sd_mask : nullptr,
                              shake ? res.sd_fwd : nullptr, res.A, res.A_lo, B, (int)res.units);
}

// The time-stepped counterparts of norm_statistics / norm_backward: statistics
// and running averages of their own per time step ([T, units] arrays), all time
// steps in one launch each.
dlb_status norm_statistics_time(dlb_model *m, LayerRT &l, const float *in, int T, int B, dlb_brn_unit_arrays *u) {
  if (m->propagation == DLB_PROPAGATION_INFERENCE) return inference_arrays(m, l, u);
  const int Bg = (int)(m->global_rows ? m->global_rows : (size_t)B);
  const int n = (int)l.norm_units;
  *u = unit_arrays(m, l, 0);
  DLB_TRY(dlb_brn_time_forward_sums(m->ctx, in, T, B, n, l.fwd_sums));
  DLB_TRY(dlb_allreduce_f64(m->ctx, l.fwd_sums, 2 * (size_t)T * n));
  return dlb_brn_time_forward_finalize(m->ctx, l.fwd_sums, Bg, T, n, m->hp.normalization_momentum_average,
                                       m->hp.normalization_epsilon, r_max_of(m, l), d_max_of(m, l), u);
}

// `e` [T, B, n] holds dA on entry and the error w.r.t. `in` on return.
dlb_status norm_backward_time(dlb_model *m, LayerRT &l, float *e, float *e_lo, const float *in, const float *act,
                              int af, int T, int B) {
  const int Bg = (int)(m->global_rows ? m->global_rows : (size_t)B);
  const int n = (int)l.norm_units;
  const size_t plane = (size_t)T * n;
  dlb_brn_unit_arrays u = unit_arrays(m, l, 0);
  DLB_TRY(dlb_indrnn_backward_walk(m->ctx, e, in, act, &u, nullptr, af, T, B, n));
  DLB_TRY(dlb_indrnn_backward_sums(m->ctx, e, in, act, &u, 0, T, B, n, l.bwd_sums));
  DLB_TRY(dlb_time_fold(m->ctx, l.bwd_sums, T, n, m->grads + gamma_index(m, l)));
  DLB_TRY(dlb_time_fold(m->ctx, l.bwd_sums + plane, T, n, m->grads + beta_index(m, l)));
  DLB_TRY(dlb_allreduce_f64(m->ctx, l.bwd_sums + 2 * plane, 2 * plane));
  return dlb_brn_time_backward_apply(m->ctx, e, e_lo, in, &u, l.bwd_sums, Bg, T, B, n);
}

// A residual block inside a time-stepped model
// (Recurrent__Forward_Pass__Residual__OpenMP and ..__Residual__Layer__OpenMP,
// v1/learner/fwp_rec_mp.cpp L:510-700): the block's FC layers have no recurrent
// connections, so all T * B rows go through each product at once; what is per
// time step are the normalization statistics, the Bernoulli masks
// (mask[t * width + unit]) and the ShakeDrop flags (flag[t * B + b],
// fwp_mp.cpp L:4935-4955), which the [T, B, width] layout turns into row flags
// of the T * B rows.
dlb_status forward_residual_time(dlb_model *m, size_t i, const float *X, const float *X_lo, int B, int T) {
  LayerRT &res = m->layers[i];
  const bool inference = m->propagation == DLB_PROPAGATION_INFERENCE;
  const int TB = T * B;
  const float *in = X, *in_lo = X_lo;
  const float *prev_sums = nullptr;
  for (size_t j = 1; j <= res.depth; ++j) {
    LayerRT &b = m->layers[i + j];
    const bool norm = b.norm != DLB_NORM_NONE;
    if (!b.block_input) {
      dlb_brn_unit_arrays u{};
      if (norm) DLB_TRY(norm_statistics_time(m, b, prev_sums, T, B, &u));
      const uint8_t *mask = nullptr;
      float keep_scale = 1.f;
      if (b.dropout != DLB_DROPOUT_NONE) {
        if (inference) {
          if (b.dropout == DLB_DROPOUT_BERNOULLI) keep_scale = b.dropout_value;
        } else {
          mask = b.mask;
          if (b.dropout == DLB_DROPOUT_BERNOULLI_INVERTED)
            keep_scale = b.dropout_value == 0.f ? 0.f : 1.f / b.dropout_value;
        }
      }
      if (norm || mask || keep_scale != 1.f)
        DLB_TRY(dlb_indrnn_forward_dropout(m->ctx, prev_sums, norm ? &u : nullptr, nullptr, b.af, mask, keep_scale,
                                           b.IN, b.IN_lo, T, B, (int)b.fan_in));
      else
        DLB_TRY(dlb_activation_forward(m->ctx, prev_sums, nullptr, b.af, nullptr, b.IN, b.IN_lo, TB, (int)b.fan_in));
      in = b.IN;
      in_lo = b.IN_lo;
    }
    const float *bias = norm ? nullptr : m->params + b.first_bias;
    DLB_TRY(dlb_fc_forward(m->ctx, in, in_lo, m->params + b.first_conn, m->params_lo + b.first_conn, bias, b.A, TB,
                           (int)b.fan_in, (int)b.units));
    prev_sums = b.A;
  }
  LayerRT &last = m->layers[i + res.depth];
  float *block = last.A;
  const bool scale = inference && res.dropout == DLB_DROPOUT_SHAKEDROP;
  if (res.norm != DLB_NORM_NONE || scale) {
    dlb_brn_unit_arrays u{};
    if (res.norm != DLB_NORM_NONE) DLB_TRY(norm_statistics_time(m, res, last.A, T, B, &u));
    DLB_TRY(dlb_indrnn_forward_dropout(m->ctx, last.A, res.norm != DLB_NORM_NONE ? &u : nullptr, nullptr,
                                       DLB_AF_LINEAR, nullptr, scale ? 1.f - res.dropout_value : 1.f, last.delta,
                                       nullptr, T, B, (int)last.units));
    block = last.delta;
  }
  const bool shake = !inference && res.dropout == DLB_DROPOUT_SHAKEDROP;
  if (shake && (!res.sd_mask || res.sd_rows < (size_t)TB)) {
    set_error("model: residual layer %zu uses ShakeDrop but no noise was set for %d rows (seq_w * rows; "
              "dlb_model_set_shakedrop_noise)", i, TB);
    return DLB_ERR_INVALID;
  }
  if (last.units != res.fan_in)
    return dlb_residual_forward_padded(m->ctx, X, (int)res.fan_in, block, (int)last.units,
                                       shake ? res.sd_mask : nullptr, shake ? res.sd_fwd : nullptr, res.A,
                                       res.A_lo, TB);
  return dlb_residual_forward(m->ctx, X, block, shake ? res.sd_mask : nullptr, shake ? res.sd_fwd : nullptr,
                              res.A, res.A_lo, TB, (int)res.units);
}

// LSTM layer forward (Recurrent__Forward_Pass__LSTM__OpenMP,
// v1/learner/fwp_rec_mp.cpp L:395-418, L:802-1526): the input sums of all time
// steps are one product over T * B rows; per time step the recurrent sums are a
// product over B rows and the cells one kernel.
dlb_status forward_lstm(dlb_model *m, LayerRT &l, const float *X, const float *X_lo, int B, int T) {
  const int I = (int)l.fan_in, C = (int)l.units, G = (int)lstm_gates(l);
  DLB_TRY(dlb_gather_rows(m->ctx, m->params, l.lstm_map_ff, l.lstm_wff, (size_t)G, I));
  DLB_TRY(dlb_gather_rows(m->ctx, m->params, l.lstm_map_rec, l.lstm_wrec, (size_t)G, C));
  DLB_TRY(dlb_gather_rows(m->ctx, m->params, l.lstm_map_bias, l.lstm_bias, (size_t)G, 1));
  DLB_TRY(dlb_gather_rows(m->ctx, m->params, l.lstm_map_peep, l.lstm_peep, (size_t)3 * C, 1));
  DLB_TRY(dlb_fc_forward(m->ctx, X, X_lo, l.lstm_wff, nullptr, nullptr, l.lstm_gin, T * B, I, G));
  const size_t sc = (size_t)B * C, sb = (size_t)B * l.blocks, sg = (size_t)B * G;
  for (int t = 0; t < T; ++t) {
    if (t > 0)
      DLB_TRY(dlb_fc_forward(m->ctx, l.A + (t - 1) * sc, nullptr, l.lstm_wrec, nullptr, nullptr, l.lstm_grec, B, C, G));
    DLB_TRY(dlb_lstm_forward_step(m->ctx, l.lstm_gin + t * sg, t ? l.lstm_grec : nullptr, l.lstm_bias, l.lstm_peep,
                                  t ? l.lstm_c + (t - 1) * sc : nullptr, l.lstm_z + t * sc, l.lstm_c + t * sc,
                                  l.lstm_ca + t * sc, l.A + t * sc, l.lstm_gi + t * sb, l.lstm_gf + t * sb,
                                  l.lstm_go + t * sb, B, (int)l.blocks, (int)l.cells));
  }
  return dlb_split_planes_2d(m->ctx, l.A, l.A_lo, T * B, C);
}

// Backward through time: l.delta holds the error of the layer's outputs from
// above; per time step, from the last, the recurrent part is added (the gates'
// errors of t + 1 times R) and the cell kernel forms the gates' errors of t.
// Then the error of the layer's inputs is one product over T * B rows.
dlb_status backward_lstm(dlb_model *m, LayerRT &l, float *below_delta, int B, int T) {
  const int I = (int)l.fan_in, C = (int)l.units, G = (int)lstm_gates(l);
  const size_t sc = (size_t)B * C, sb = (size_t)B * l.blocks, sg = (size_t)B * G;
  for (int t = T - 1; t >= 0; --t) {
    const bool last = t == T - 1;
    float *dH = l.delta + t * sc;
    if (!last) {
      // dH_t += D_{t+1} Wrec  (Backward_Pass__LSTM_Derivative__Output, bwp_rec_mp.cpp L:1160-1196)
      GemmOperand A{l.lstm_d + (t + 1) * sg, nullptr, (long long)G, 1};
      GemmOperand Bo{l.lstm_wrec, nullptr, 1, (long long)C};
      GemmEpilogue ep;
      ep.accumulate = 1;
      DLB_TRY(gemm(m->ctx, A, Bo, dH, (long long)C, B, C, G, ep));
    }
    float *dC = l.lstm_dc + (size_t)(t & 1) * sc, *dC_next = l.lstm_dc + (size_t)((t + 1) & 1) * sc;
    DLB_TRY(dlb_lstm_backward_step(m->ctx, dH, l.lstm_z + t * sc, l.lstm_ca + t * sc, l.lstm_gi + t * sb,
                                   l.lstm_gf + t * sb, l.lstm_go + t * sb, t ? l.lstm_c + (t - 1) * sc : nullptr,
                                   last ? nullptr : l.lstm_gf + (t + 1) * sb, last ? nullptr : dC_next,
                                   last ? nullptr : l.lstm_d + (t + 1) * sg, l.lstm_peep, dC, l.lstm_d + t * sg, B,
                                   (int)l.blocks, (int)l.cells));
  }
  if (below_delta)
    DLB_TRY(dlb_fc_backward_input(m->ctx, l.lstm_d, nullptr, l.lstm_wff, nullptr, below_delta, T * B, I, G));
  return DLB_OK;
}

// Weight gradients of an LSTM layer in packed form, scattered (added) into the
// gradient vector; the bias gradients wait in l.lstm_dbias for the end of the
// pass (their indices reach into the next layer's biases, which that layer's
// own gradient would overwrite).
dlb_status derivatives_lstm(dlb_model *m, LayerRT &l, const float *X, const float *X_lo, int B, int T) {
  const int I = (int)l.fan_in, C = (int)l.units, G = (int)lstm_gates(l);
  const size_t sg = (size_t)B * G;
  // dWff = D^T X over all T * B rows, with the column sums of D as bias gradient.
  DLB_TRY(dlb_fc_weight_gradient(m->ctx, l.lstm_d, nullptr, X, X_lo, l.lstm_dwff, l.lstm_dbias, T * B, I, G, 0));
  DLB_TRY(dlb_scatter_add_rows(m->ctx, l.lstm_dwff, l.lstm_map_ff, m->grads, (size_t)G, I));
  if (T > 1) {
    // dWrec = sum_t D_{t+1}^T h_t (update_derivative_rec_mp.cpp L:571-575, L:616-622).
    DLB_TRY(dlb_fc_weight_gradient(m->ctx, l.lstm_d + sg, nullptr, l.A, l.A_lo, l.lstm_dwrec, nullptr, (T - 1) * B,
                                   C, G, 0));
    DLB_TRY(dlb_scatter_add_rows(m->ctx, l.lstm_dwrec, l.lstm_map_rec, m->grads, (size_t)G, C));
  }
  DLB_TRY(dlb_lstm_peephole_gradient(m->ctx, l.lstm_d, l.lstm_c, l.lstm_dpeep, T, B, (int)l.blocks, (int)l.cells));
  return dlb_scatter_add_rows(m->ctx, l.lstm_dpeep, l.lstm_map_peep, m->grads, (size_t)3 * C, 1);
}

// Time-stepped forward, layer-major as the reference
// (RNN__Forward_Pass_Batch__OpenMP, v1/learner/fwp_rec_mp.cpp L:29-110): one
// GEMM over all T * rows rows of a layer, statistics for every time step in one
// launch, then the walk over time.
dlb_status forward_layers_time(dlb_model *m, size_t rows) {
  DLB_TRY(refresh_weight_residuals(m));
  const int B = (int)rows, T = (int)m->seq_w;
  const int TB = T * B;
  const int Bg = (int)(m->global_rows ? m->global_rows : rows);
  const float *X = m->input, *X_lo = m->input_lo;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) {
      DLB_TRY(forward_residual_time(m, i, X, X_lo, B, T));
      X = l.A;
      X_lo = l.A_lo;
      i += l.depth;
      continue;
    }
    if (is_lstm(l)) {
      DLB_TRY(forward_lstm(m, l, X, X_lo, B, T));
      X = l.A;
      X_lo = l.A_lo;
      continue;
    }
    const int I = (int)l.fan_in, H = (int)l.units;
    const bool norm = l.norm != DLB_NORM_NONE;
    const bool last = i + 1 == m->layers.size();
    const float *bias = norm ? nullptr : m->params + l.first_bias;
    DLB_TRY(dlb_fc_forward(m->ctx, X, X_lo, m->params + l.first_conn, m->params_lo + l.first_conn,
                           bias, l.Z, TB, I, H));
    if (l.af == DLB_AF_SOFTMAX) {
      DLB_TRY(dlb_softmax_forward(m->ctx, l.Z, l.A, TB, H));
    } else if (norm || is_indrnn(l) || l.dropout != DLB_DROPOUT_NONE) {
      dlb_brn_unit_arrays u{};
      if (norm && m->propagation == DLB_PROPAGATION_INFERENCE) {
        DLB_TRY(inference_arrays(m, l, &u));  // every time step has its own running averages
      } else if (norm) {
        u = unit_arrays(m, l, 0);
        DLB_TRY(dlb_brn_time_forward_sums(m->ctx, l.Z, T, B, H, l.fwd_sums));
        DLB_TRY(dlb_allreduce_f64(m->ctx, l.fwd_sums, 2 * (size_t)T * H));
        DLB_TRY(dlb_brn_time_forward_finalize(m->ctx, l.fwd_sums, Bg, T, H,
                                              m->hp.normalization_momentum_average,
                                              m->hp.normalization_epsilon, r_max_of(m, l),
                                              d_max_of(m, l), &u));
      }
      // Dropout of time step t acts on the stored output, which the recurrence
      // of step t + 1 reads; at inference the plain form scales by the keep
      // probability and the inverted form does nothing.
      const uint8_t *mask = nullptr;
      float keep_scale = 1.f;
      if (l.dropout != DLB_DROPOUT_NONE && !last) {
        if (m->propagation == DLB_PROPAGATION_INFERENCE) {
          if (l.dropout == DLB_DROPOUT_BERNOULLI) keep_scale = l.dropout_value;
        } else {
          mask = l.mask;
          if (l.dropout == DLB_DROPOUT_BERNOULLI_INVERTED)
            keep_scale = l.dropout_value == 0.f ? 0.f : 1.f / l.dropout_value;
        }
      }
      if (l.dropout == DLB_DROPOUT_UOUT && !last && m->propagation != DLB_PROPAGATION_INFERENCE) {
        // Draws for all T * B rows, [T, B, H] (an input of the step like the masks).
        DLB_TRY(uout_ready(m, l, i, TB));
        DLB_TRY(dlb_indrnn_forward_uout(m->ctx, l.Z, norm ? &u : nullptr,
                                        is_indrnn(l) ? m->params + l.first_recurrent : nullptr, l.af, l.uout, l.A,
                                        l.A_lo, T, B, H));
      } else {
        DLB_TRY(dlb_indrnn_forward_dropout(m->ctx, l.Z, norm ? &u : nullptr,
                                           is_indrnn(l) ? m->params + l.first_recurrent : nullptr, l.af, mask,
                                           keep_scale, l.A, last ? nullptr : l.A_lo, T, B, H));
      }
    } else {
      DLB_TRY(dlb_activation_forward(m->ctx, l.Z, nullptr, l.af, nullptr, l.A, last ? nullptr : l.A_lo,
                                     TB, H));
    }
    X = l.A;
    X_lo = l.A_lo;
  }
  return DLB_OK;
}

dlb_status forward_layers(dlb_model *m, size_t rows) {
  const bool inference = m->propagation == DLB_PROPAGATION_INFERENCE;
  if (time_stepped(m)) return forward_layers_time(m, rows);
  DLB_TRY(refresh_weight_residuals(m));
  const int B = (int)rows;
  const float *X = m->input, *X_lo = m->input_lo;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) {
      DLB_TRY(forward_residual(m, i, X, X_lo, B));
      X = l.A;
      X_lo = l.A_lo;
      i += l.depth;
      continue;
    }
    const int I = (int)l.fan_in, H = (int)l.units;
    const bool norm = l.norm != DLB_NORM_NONE;
    const bool last = i + 1 == m->layers.size();
    // The bias enters only where there is no normalisation (model.hpp L:708).
    const float *bias = norm ? nullptr : m->params + l.first_bias;
    if (!norm && !last && !inference && l.af != DLB_AF_SOFTMAX) {
      // A hidden layer without normalization: bias, activation and dropout ride
      // in the product's epilogue (where the kernel that runs has one).
      DLB_TRY(uout_ready(m, l, i, B));
      dlb_dropout_desc dp{l.dropout, l.dropout_value, l.mask, l.uout};
      DLB_TRY(dlb_fc_forward_activation(m->ctx, X, X_lo, m->params + l.first_conn, m->params_lo + l.first_conn,
                                        bias, l.Z, l.af, l.dropout != DLB_DROPOUT_NONE ? &dp : nullptr, l.A,
                                        l.A_lo, B, I, H));
      X = l.A;
      X_lo = l.A_lo;
      continue;
    }
    DLB_TRY(dlb_fc_forward(m->ctx, X, X_lo, m->params + l.first_conn, m->params_lo + l.first_conn,
                           bias, l.Z, B, I, H));
    dlb_brn_unit_arrays u;
    if (norm) DLB_TRY(norm_statistics(m, l, l.Z, B, &u));
    if (l.af == DLB_AF_SOFTMAX) {
      DLB_TRY(dlb_softmax_forward(m->ctx, l.Z, l.A, B, H));
    } else if (inference) {
      // Plain Bernoulli dropout scales by the keep probability at inference
      // (fwp_mp.cpp L:4870-4892); the other kinds do nothing.
      dlb_dropout_desc dp{DROPOUT_INFERENCE_SCALE, l.dropout_value, nullptr, nullptr};
      DLB_TRY(dlb_activation_forward(m->ctx, l.Z, norm ? &u : nullptr, l.af,
                                     l.dropout == DLB_DROPOUT_BERNOULLI ? &dp : nullptr, l.A,
                                     last ? nullptr : l.A_lo, B, H));
    } else {
      DLB_TRY(uout_ready(m, l, i, B));
      dlb_dropout_desc dp{l.dropout, l.dropout_value, l.mask, l.uout};
      DLB_TRY(dlb_activation_forward(m->ctx, l.Z, norm ? &u : nullptr, l.af,
                                     l.dropout != DLB_DROPOUT_NONE ? &dp : nullptr, l.A,
                                     last ? nullptr : l.A_lo, B, H));
    }
    X = l.A;
    X_lo = l.A_lo;
  }
  return DLB_OK;
}

}  // namespace

HostWorkers::HostWorkers(size_t threads) {
  for (size_t i = 0; i < threads; ++i) threads_.emplace_back([this] { loop(); });
}

HostWorkers::~HostWorkers() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    stop_ = true;
  }
  work_.notify_all();
  for (std::thread &t : threads_) t.join();
}

void HostWorkers::loop() {
  std::unique_lock<std::mutex> lock(mu_);
  for (;;) {
    work_.wait(lock, [this] { return stop_ || (fn_ && next_ < parts_); });
    if (stop_) return;
    const size_t part = next_++;
    const std::function<void(size_t)> *fn = fn_;
    lock.unlock();
    (*fn)(part);
    lock.lock();
    if (++finished_ == parts_) done_.notify_all();
  }
}

void HostWorkers::run(size_t parts, const std::function<void(size_t)> &fn) {
  if (parts == 0) return;
  std::unique_lock<std::mutex> lock(mu_);
  fn_ = &fn;
  parts_ = parts;
  next_ = finished_ = 0;
  work_.notify_all();
  // The caller takes parts as well.
  while (next_ < parts_) {
    const size_t part = next_++;
    lock.unlock();
    fn(part);
    lock.lock();
    ++finished_;
  }
  done_.wait(lock, [this] { return finished_ == parts_; });
  fn_ = nullptr;
}

namespace {

// Host rows (the reference's array of row pointers, pageable memory) into a
// device tensor: gathered into a page-locked staging buffer by a few host
// threads that the model keeps, piece by piece; the thread that completes a
// piece starts its copy to the device, which runs while the next pieces are
// gathered.  The copies run on the copy stream, so that the
// targets of a step cross while its forward pass computes; the compute stream
// waits for them where it needs them (rows_staged).  which: 0 inputs, 1 targets.
dlb_status stage_rows(dlb_model *m, int which, float **stage, size_t *stage_elems, size_t rows, size_t width,
                      const float *const *row_ptrs, float *dev) {
  DLB_CUDA(cudaSetDevice(m->ctx->device));
  if (!m->copy_stream) DLB_CUDA(cudaStreamCreateWithFlags(&m->copy_stream, cudaStreamNonBlocking));
  if (!m->rows_copied[which]) {
    DLB_CUDA(cudaEventCreateWithFlags(&m->rows_copied[which], cudaEventDisableTiming));
    DLB_CUDA(cudaEventCreateWithFlags(&m->rows_consumed[which], cudaEventDisableTiming));
  }
  // The previous copy out of this staging buffer must have finished, also
  // before the buffer is replaced by a larger one.
  if (m->rows_in_flight[which]) DLB_CUDA(cudaEventSynchronize(m->rows_copied[which]));
  const size_t need = rows * width;
  if (need > *stage_elems) {
    if (*stage) DLB_TRY(dlb_host_free(*stage));
    *stage = nullptr;
    DLB_TRY(dlb_host_alloc(reinterpret_cast<void **>(stage), need * sizeof(float)));
    *stage_elems = need;
  }
  // The kernels that read the device tensor last must be past it.
  if (m->rows_in_flight[which]) DLB_CUDA(cudaStreamWaitEvent(m->copy_stream, m->rows_consumed[which], 0));
  else DLB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  constexpr size_t PIECE_BYTES = 2u << 20;
  const size_t piece_rows = std::max<size_t>(1, PIECE_BYTES / (width * sizeof(float)));
  const size_t pieces = (rows + piece_rows - 1) / piece_rows;
  if (need * sizeof(float) < (1u << 20)) {
    for (size_t r = 0; r < rows; ++r) memcpy(*stage + r * width, row_ptrs[r], width * sizeof(float));
    DLB_CUDA(cudaMemcpyAsync(dev, *stage, need * sizeof(float), cudaMemcpyHostToDevice, m->copy_stream));
  } else {
    if (!m->workers) {
      const unsigned hw = std::thread::hardware_concurrency();
      m->workers = new HostWorkers(std::min<size_t>(8, hw ? hw : 1) - 1);
    }
    // Every piece is split among `split` threads; the one that finishes a piece
    // last sends it.
    const size_t split = std::min<size_t>(m->workers->size(), 4);
    std::vector<std::atomic<int>> left(pieces);
    for (auto &a : left) a.store((int)split);
    std::atomic<int> failed{0};
    float *staging = *stage;
    const int device = m->ctx->device;
    cudaStream_t copy_stream = m->copy_stream;
    m->workers->run(pieces * split, [&](size_t part) {
      const size_t piece = part / split, share = part % split;
      const size_t r0 = piece * piece_rows, r1 = std::min(rows, r0 + piece_rows);
      const size_t per = (r1 - r0 + split - 1) / split;
      const size_t a = std::min(r1, r0 + share * per), b = std::min(r1, a + per);
      for (size_t r = a; r < b; ++r) memcpy(staging + r * width, row_ptrs[r], width * sizeof(float));
      if (left[piece].fetch_sub(1) == 1) {
        if (cudaSetDevice(device) != cudaSuccess ||
            cudaMemcpyAsync(dev + r0 * width, staging + r0 * width, (r1 - r0) * width * sizeof(float),
                            cudaMemcpyHostToDevice, copy_stream) != cudaSuccess)
          failed.store(1);
      }
    });
    if (failed.load()) {
      set_error("stage_rows: copy to the device failed: %s", cudaGetErrorString(cudaGetLastError()));
      return DLB_ERR_CUDA;
    }
  }
  DLB_CUDA(cudaEventRecord(m->rows_copied[which], m->copy_stream));
  DLB_CUDA(cudaStreamWaitEvent(m->ctx->stream, m->rows_copied[which], 0));
  m->rows_in_flight[which] = true;
  return DLB_OK;
}

// After the kernels that read a tensor filled by stage_rows have been enqueued.
dlb_status rows_consumed(dlb_model *m, int which) {
  if (m->rows_in_flight[which]) DLB_CUDA(cudaEventRecord(m->rows_consumed[which], m->ctx->stream));
  return DLB_OK;
}

dlb_status stage_block(dlb_model *m, float **stage, size_t *stage_elems, size_t elems,
                       const float *host, float *dev) {
  cudaPointerAttributes attr;
  const bool pinned = cudaPointerGetAttributes(&attr, host) == cudaSuccess &&
                      attr.type == cudaMemoryTypeHost;
  cudaGetLastError();
  if (pinned) return dlb_memcpy_h2d(m->ctx, dev, host, elems * sizeof(float));
  if (elems > *stage_elems) {
    if (*stage) DLB_TRY(dlb_host_free(*stage));
    *stage = nullptr;
    DLB_TRY(dlb_host_alloc(reinterpret_cast<void **>(stage), elems * sizeof(float)));
    *stage_elems = elems;
  }
  DLB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  memcpy(*stage, host, elems * sizeof(float));
  return dlb_memcpy_h2d(m->ctx, dev, *stage, elems * sizeof(float));
}

LayerRT *layer_at(dlb_model *m, size_t i) { return i < m->layers.size() ? &m->layers[i] : nullptr; }

float *named_array(dlb_model *m, const std::string &n) {
  if (n == "parameters") return m->params;
  if (n == "derivatives") return m->grads;
  if (n == "first_moment") return m->m1;
  if (n == "second_moment") return m->m2;
  if (n == "second_moment_hat") return m->m2hat;
  return nullptr;
}

int norm_field(const std::string &n) {
  if (n == "mean") return 0;
  if (n == "variance") return 1;  // the reference's "variance" arrays hold sigma
  if (n == "mean_average") return 2;
  if (n == "variance_average") return 3;
  if (n == "r_correction") return 4;
  if (n == "d_correction") return 5;
  return -1;
}

}  // namespace

extern "C" {

dlb_status dlb_model_create(dlb_model **out, dlb_ctx *ctx) {
  DLB_REQUIRE(out && ctx, "dlb_model_create: null");
  *out = new dlb_model;
  (*out)->ctx = ctx;
  return DLB_OK;
}

dlb_status dlb_model_destroy(dlb_model *m) {
  if (!m) return DLB_OK;
  free_batch_buffers(m);
  for (auto &l : m->layers) {
    if (l.stats) dlb_free(m->ctx, l.stats);
    if (l.mask) dlb_free(m->ctx, l.mask);
    if (l.uout) dlb_free(m->ctx, l.uout);
    if (l.sd_mask) dlb_free(m->ctx, l.sd_mask);
    if (l.sd_fwd) dlb_free(m->ctx, l.sd_fwd);
    if (l.sd_bwd) dlb_free(m->ctx, l.sd_bwd);
    if (l.fwd_sums) dlb_free(m->ctx, l.fwd_sums);
    if (l.bwd_sums) dlb_free(m->ctx, l.bwd_sums);
    if (l.ev_reduced) cudaEventDestroy(l.ev_reduced);
    if (l.ev_gathered) cudaEventDestroy(l.ev_gathered);
    void *lstm[] = {l.lstm_wff, l.lstm_wrec, l.lstm_bias, l.lstm_peep, l.lstm_dwff, l.lstm_dwrec, l.lstm_dbias,
                    l.lstm_dpeep, l.lstm_map_ff, l.lstm_map_rec, l.lstm_map_bias, l.lstm_map_peep};
    for (void *p : lstm)
      if (p) dlb_free(m->ctx, p);
  }
  float *flat[] = {m->params, m->params_lo, m->grads, m->m1, m->m2, m->m2hat, m->wd_mask};
  for (float *p : flat)
    if (p) dlb_free(m->ctx, p);
  if (m->loss_sum) dlb_free(m->ctx, m->loss_sum);
  if (m->loss_tmp) dlb_free(m->ctx, m->loss_tmp);
  if (m->loss_host) dlb_host_free(m->loss_host);
  for (cudaEvent_t e : m->loss_ready)
    if (e) cudaEventDestroy(e);
  if (m->accu_sum) dlb_free(m->ctx, m->accu_sum);
  if (m->ones) dlb_free(m->ctx, m->ones);
  if (m->zeros) dlb_free(m->ctx, m->zeros);
  delete m->workers;
  if (m->copy_stream) {
    cudaStreamSynchronize(m->copy_stream);
    cudaStreamDestroy(m->copy_stream);
  }
  if (m->stage_x) dlb_host_free(m->stage_x);
  if (m->stage_y) dlb_host_free(m->stage_y);
  for (int w = 0; w < 2; ++w) {
    if (m->rows_copied[w]) cudaEventDestroy(m->rows_copied[w]);
    if (m->rows_consumed[w]) cudaEventDestroy(m->rows_consumed[w]);
  }
  for (auto &a : m->ahead) {
    if (a.x) dlb_free(m->ctx, a.x);
    if (a.y) dlb_free(m->ctx, a.y);
    if (a.ready) cudaEventDestroy(a.ready);
    if (a.consumed) cudaEventDestroy(a.consumed);
  }
  delete m;
  return DLB_OK;
}

dlb_status dlb_model_compile(dlb_model *m, size_t n_layers, size_t seq_w, int model_type,
                             const int *layer_types, const size_t *layer_units) {
  return dlb_model_compile2(m, n_layers, seq_w, model_type, layer_types, layer_units, nullptr);
}

// layer_units2: Layer_Parameters::unit_parameters[1], the cells per block of an
// LSTM layer (its unit_parameters[0] being the number of blocks; compile.cpp L:98-118).
dlb_status dlb_model_compile2(dlb_model *m, size_t n_layers, size_t seq_w, int model_type,
                              const int *layer_types, const size_t *layer_units, const size_t *layer_units2) {
  DLB_REQUIRE(m && layer_types && layer_units && n_layers >= 2 && seq_w >= 1, "dlb_model_compile");
  DLB_REQUIRE(m->layers.empty(), "dlb_model_compile: already compiled");
  DLB_REQUIRE(layer_types[0] == DLB_LAYER_FULLY_CONNECTED &&
                  layer_types[n_layers - 1] == DLB_LAYER_FULLY_CONNECTED,
              "dlb_model_compile: input and output layers are fully connected layers");
  for (size_t i = 0; i < n_layers; ++i)
    DLB_REQUIRE(layer_units[i] > 0, "dlb_model_compile: empty layer");
  m->layers.resize(n_layers);
  for (size_t i = 0; i < n_layers; ++i) {
    m->layers[i].type = layer_types[i];
    // For a RESIDUAL layer the parameter is the block depth (model.hpp L:78-82).
    if (layer_types[i] == DLB_LAYER_RESIDUAL) {
      m->layers[i].depth = layer_units[i];
    } else if (layer_types[i] == DLB_LAYER_LSTM) {
      if (!layer_units2 || layer_units2[i] == 0) {
        m->layers.clear();
        set_error("dlb_model_compile: LSTM layer %zu needs its cells per block (dlb_model_compile2)", i);
        return DLB_ERR_INVALID;
      }
      m->layers[i].blocks = layer_units[i];
      m->layers[i].cells = layer_units2[i];
      m->layers[i].units = layer_units[i] * layer_units2[i];
    } else {
      m->layers[i].units = layer_units[i];
    }
  }
  m->seq_w = seq_w;
  m->model_type = model_type;
  const dlb_status st = layout_parameters(m);
  if (st != DLB_OK) m->layers.clear();
  return st;
}

dlb_status dlb_model_set_layer_activation_function(dlb_model *m, size_t layer, int af) {
  DLB_REQUIRE(m && layer_at(m, layer) && layer > 0, "set_layer_activation_function: bad layer");
  if (!af_supported(af)) {
    set_error("set_layer_activation_function: activation %d is outside the supported set", af);
    return DLB_ERR_UNSUPPORTED;
  }
  m->layers[layer].af = af;
  return DLB_OK;
}

dlb_status dlb_model_set_layer_normalization(dlb_model *m, size_t layer, int norm) {
  DLB_REQUIRE(m && layer_at(m, layer), "Set__Layer_Normalization: bad layer");
  // Not on the input or output layer (v1/learner/normalization.cpp L:419-422).
  DLB_REQUIRE(layer > 0 && layer + 1 < m->layers.size(),
              "Set__Layer_Normalization: not available on the input or output layer");
  if (norm != DLB_NORM_NONE && norm != DLB_NORM_BATCH_RENORMALIZATION && norm != DLB_NORM_BATCH_NORMALIZATION) {
    set_error("Set__Layer_Normalization: batch normalization and renormalization are supported (got %d)", norm);
    return DLB_ERR_UNSUPPORTED;
  }
  if (m->layers[layer].stats) {
    set_error("Set__Layer_Normalization: cannot change after the first training step");
    return DLB_ERR_UNSUPPORTED;
  }
  m->layers[layer].norm = norm;
  if (m->params) return allocate_parameters(m);
  return layout_parameters(m);
}

dlb_status dlb_model_set_dropout(dlb_model *m, size_t layer, int type, float value0,
                                 int scale_weights) {
  DLB_REQUIRE(m && layer_at(m, layer), "set_dropout: bad layer");
  // Not on the output layer (v1/learner/dropout.cpp L:57-60).
  DLB_REQUIRE(layer + 1 < m->layers.size(), "set_dropout: not available on the output layer");
  const bool residual = m->layers[layer].type == DLB_LAYER_RESIDUAL;
  if (residual) {
    // A residual layer takes ShakeDrop only; value0 is the probability that a
    // row IS perturbed (fwp_mp.cpp L:4942-4955).
    if (type != DLB_DROPOUT_NONE && type != DLB_DROPOUT_SHAKEDROP) {
      set_error("set_dropout: a residual layer supports ShakeDrop only (got %d)", type);
      return DLB_ERR_UNSUPPORTED;
    }
    if (type != DLB_DROPOUT_NONE) DLB_REQUIRE(value0 >= 0.f && value0 <= 1.f, "set_dropout: probability");
  } else {
    if (type != DLB_DROPOUT_NONE && type != DLB_DROPOUT_BERNOULLI &&
        type != DLB_DROPOUT_BERNOULLI_INVERTED && type != DLB_DROPOUT_UOUT) {
      set_error("set_dropout: dropout type %d is outside the supported set of this build", type);
      return DLB_ERR_UNSUPPORTED;
    }
    // Bernoulli: keep probability; UOut: half-width beta of the noise U(-beta, beta).
    if (type != DLB_DROPOUT_NONE) DLB_REQUIRE(value0 > 0.f && value0 <= 1.f, "set_dropout: value in (0, 1]");
    // The input layer's dropout acts on the batch as it is assigned
    // (v1/learner/assign_inputs.cpp L:94-130); the Bernoulli kinds are built.
    if (layer == 0 && type == DLB_DROPOUT_UOUT) {
      set_error("set_dropout: UOut on the input layer is outside the supported path");
      return DLB_ERR_UNSUPPORTED;
    }
  }
  if (scale_weights) {
    set_error("set_dropout: scale_weights=true is not supported (on a fresh layer the reference "
              "multiplies the layer's weights by 0/keep); pass false");
    return DLB_ERR_UNSUPPORTED;
  }
  m->layers[layer].dropout = type;
  m->layers[layer].dropout_value = value0;
  return DLB_OK;
}

dlb_status dlb_model_set_normalization_momentum_average(dlb_model *m, float v) {
  DLB_REQUIRE(m, "null");
  m->hp.normalization_momentum_average = v;
  return DLB_OK;
}
dlb_status dlb_model_set_normalization_epsilon(dlb_model *m, float v) {
  DLB_REQUIRE(m, "null");
  m->hp.normalization_epsilon = v;
  return DLB_OK;
}
dlb_status dlb_model_set_brn_r_correction_maximum(dlb_model *m, float v) {
  DLB_REQUIRE(m, "null");
  m->hp.brn_r_max = v;
  return DLB_OK;
}
dlb_status dlb_model_set_brn_d_correction_maximum(dlb_model *m, float v) {
  DLB_REQUIRE(m, "null");
  m->hp.brn_d_max = v;
  return DLB_OK;
}

dlb_status dlb_model_set_loss_fn(dlb_model *m, int loss) {
  DLB_REQUIRE(m, "null");
  if (loss != DLB_LOSS_MSE && loss != DLB_LOSS_CROSS_ENTROPY) {
    set_error("set_loss_fn: loss %d is outside the supported set (MSE, CROSS_ENTROPY)", loss);
    return DLB_ERR_UNSUPPORTED;
  }
  m->loss = loss;
  return DLB_OK;
}

dlb_status dlb_model_set_optimizer(dlb_model *m, int optimizer) {
  DLB_REQUIRE(m, "null");
  switch (optimizer) {
    case DLB_OPT_ADABOUND: case DLB_OPT_ADAM: case DLB_OPT_ADAMAX: case DLB_OPT_AMSBOUND:
    case DLB_OPT_AMSGRAD: case DLB_OPT_NOSADAM: case DLB_OPT_GD:
      m->optimizer = optimizer;
      return DLB_OK;
    default:
      set_error("set_optimizer: optimizer %d is outside the supported set", optimizer);
      return DLB_ERR_UNSUPPORTED;
  }
}

#define DLB_HPARAMS(X)                                                                       \
  X(adam_learning_rate) X(adam_beta1) X(adam_beta2) X(adam_previous_beta2) X(adam_epsilon)   \
  X(adam_gamma) X(learning_rate_final) X(learning_gamma) X(weight_decay)                     \
  X(optimizer_time_step) X(epoch_time_step) X(learning_rate) X(learning_momentum)

dlb_status dlb_model_set_hparam(dlb_model *m, const char *name, double value) {
  DLB_REQUIRE(m && name, "set_hparam: null");
  const std::string n(name);
#define X(f) if (n == #f) { m->hp.f = (float)value; return DLB_OK; }
  DLB_HPARAMS(X)
#undef X
  if (n == "use_adam_bias_correction") { m->hp.use_adam_bias_correction = value != 0.0; return DLB_OK; }
  if (n == "use_nesterov") { m->hp.use_nesterov = value != 0.0; return DLB_OK; }
  if (n == "use_normalized_weight_decay") { m->hp.use_normalized_weight_decay = value != 0.0; return DLB_OK; }
  if (n == "pct_threads") return DLB_OK;  // CPU threading knob of the reference; nothing to set
  set_error("set_hparam: unknown field %s", name);
  return DLB_ERR_INVALID;
}

double dlb_model_get_hparam(dlb_model *m, const char *name) {
  if (!m || !name) return -1.0;
  const std::string n(name);
#define X(f) if (n == #f) return (double)m->hp.f;
  DLB_HPARAMS(X)
#undef X
  if (n == "use_adam_bias_correction") return m->hp.use_adam_bias_correction;
  if (n == "use_nesterov") return m->hp.use_nesterov;
  if (n == "use_normalized_weight_decay") return m->hp.use_normalized_weight_decay;
  return -1.0;
}

// ref: Model::set_weight_decay (v1/ops/regularizers/weight_decay.cpp L:26-60).
dlb_status dlb_model_set_weight_decay(dlb_model *m, float value) {
  DLB_REQUIRE(m && value >= 0.f && value <= 1.f, "set_weight_decay: value in [0, 1]");
  m->hp.weight_decay = value;
  return DLB_OK;
}

// ref: Model::set_l2 (v1/ops/regularizers/l2.cpp L:31-66).  The value is kept (it
// is part of the hyperparameter file) and, as in the reference, never reaches the
// gradient: update_weights_mp calls the L2 routine with (batch_size, 0,
// total_weights) where it takes (start, end, batch_size) (v1/learner/model.cpp
// L:4717-4719, l2.cpp L:92-104), so its loop covers no element.
dlb_status dlb_model_set_l2(dlb_model *m, float value) {
  DLB_REQUIRE(m && value >= 0.f && value <= 1.f, "set_l2: value in [0, 1]");
  m->hp.regularization_l2 = value;
  return DLB_OK;
}

dlb_status dlb_model_set_max_batch_size(dlb_model *m, size_t rows) {
  DLB_REQUIRE(m && rows > 0, "set_max_batch_size");
  m->max_batch = rows;
  return DLB_OK;
}

dlb_status dlb_model_set_seq_w(dlb_model *m, size_t time_delays) {
  DLB_REQUIRE(m && time_delays < m->seq_w, "set_seq_w");
  m->n_time_delay = time_delays;
  return DLB_OK;
}

dlb_status dlb_model_seed_weights(dlb_model *m, unsigned seed) {
  DLB_REQUIRE(m, "null");
  m->weight_seed = seed;
  m->weight_gen.seed(seed);
  return DLB_OK;
}

// Glorot-uniform draw in parameter order from std::mt19937 through
// std::uniform_real_distribution<float>, bias 0.
// ref: Model::initialize_weights_with_glorot_uniform (v1/ops/initializers/glorot.cpp
// L:27-108, L:226-277).  fan_out is the width of the next layer, and for the
// output layer fan_out := fan_in.
dlb_status dlb_model_initialize_weights_with_glorot_uniform(dlb_model *m) {
  DLB_REQUIRE(m && m->layers.size() >= 2, "glorot: compile first");
  if (!m->params) DLB_TRY(allocate_parameters(m));
  std::vector<float> w(m->total_weights + m->total_bias, 0.f);
  std::uniform_real_distribution<float> dist;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;  // no weights of its own
    const size_t fan_in = l.fan_in;
    const size_t fan_out = i + 1 < m->layers.size() ? m->layers[i + 1].units : fan_in;
    float gain = 1.f, bound;
    const bool rect = l.af == DLB_AF_RELU || l.af == DLB_AF_LEAKY_RELU || l.af == DLB_AF_SELU;
    if (l.af == DLB_AF_RELU) gain = sqrtf(2.f);
    if (l.af == DLB_AF_LEAKY_RELU) gain = sqrtf(2.f / (1.f + powf(0.01f, 2.f)));
    if (rect) bound = sqrtf(6.f / (float)fan_in);
    else bound = sqrtf(6.f / (float)(fan_in + fan_out));
    bound *= gain;
    dist.param(std::uniform_real_distribution<float>::param_type(-bound, bound));
    for (size_t k = l.first_conn; k < l.last_conn; ++k) w[k] = dist(m->weight_gen);
    if (is_indrnn(l)) {
      // The recurrent weights are drawn again from U(0, mag^(1/T))
      // (Model::indrec_initialize_uniform, v1/learner/model.cpp L:5289-5333).
      const float top = powf(indrnn_magnitude(m), 1.f / (float)m->seq_w);
      dist.param(std::uniform_real_distribution<float>::param_type(-0.f, top));
      for (size_t k = 0; k < l.units; ++k) w[l.first_recurrent + k] = dist(m->weight_gen);
    }
  }
  // With the error on the last time step only, the top IndRNN layer's recurrent
  // weights are drawn once more from U((1/mag)^(1/T), mag^(1/T)) to keep long-term
  // memory (Model::indrec_initialize_uniform_ltm, model.cpp L:5335-5400).
  if (m->seq_w > 1 && m->n_time_delay + 1 == m->seq_w) {
    for (size_t i = m->layers.size() - 2; i >= 1; --i) {
      const LayerRT &l = m->layers[i];
      if (!is_indrnn(l)) continue;
      const float T = (float)m->seq_w;
      const float mag = indrnn_magnitude(m);
      dist.param(std::uniform_real_distribution<float>::param_type(powf(1.f / mag, 1.f / T),
                                                                   powf(mag, 1.f / T)));
      for (size_t k = 0; k < l.units; ++k) w[l.first_recurrent + k] = dist(m->weight_gen);
      break;
    }
  }
  DLB_TRY(dlb_memcpy_h2d(m->ctx, m->params, w.data(), w.size() * sizeof(float)));
  DLB_TRY(dlb_ctx_sync(m->ctx, nullptr));
  m->params_lo_valid = false;
  return DLB_OK;
}

size_t dlb_model_get_size(dlb_model *m, const char *name) {
  if (!m || !name) return (size_t)-1;
  const std::string n(name);
  if (n == "total_parameters") return m->total_parameters;
  if (n == "total_weights") return m->total_weights;
  if (n == "total_bias") return m->total_bias;
  if (n == "total_layers") return m->layers.size();
  if (n == "total_normalized_units") return m->total_norm_units;
  if (n == "number_threads") return 1;
  if (n == "batch_size") return m->alloc_rows ? m->alloc_rows : m->max_batch;
  if (n == "seq_w") return m->seq_w;
  if (n == "n_time_delay") return m->n_time_delay;
  if (n == "n_inp") return m->layers.empty() ? 0 : n_in(m);
  if (n == "n_out") return m->layers.empty() ? 0 : n_out(m);
  return (size_t)-1;
}

dlb_status dlb_model_layer_info(dlb_model *m, size_t layer, size_t out[10]) {
  DLB_REQUIRE(m && out && layer_at(m, layer), "layer_info");
  const LayerRT &l = m->layers[layer];
  out[0] = (size_t)l.type;
  out[1] = l.units;
  out[2] = l.first_conn;
  out[3] = l.last_conn;
  out[4] = l.first_bias;
  out[5] = l.last_bias;
  out[6] = (size_t)l.norm;
  out[7] = (size_t)l.dropout;
  out[8] = (size_t)l.group;
  out[9] = m->any_norm ? l.first_norm_unit : 0;
  return DLB_OK;
}

static dlb_status gather_moments(dlb_model *m);

dlb_status dlb_model_get_array(dlb_model *m, const char *name, float *host_out, size_t n) {
  DLB_REQUIRE(m && name && host_out, "get_array: null");
  if (!m->params) DLB_TRY(allocate_parameters(m));
  float *p = named_array(m, name);
  DLB_REQUIRE(p && n <= m->total_parameters, "get_array: unknown name or size");
  if (p == m->m1 || p == m->m2 || p == m->m2hat) DLB_TRY(gather_moments(m));
  return dlb_memcpy_d2h(m->ctx, host_out, p, n * sizeof(float));
}

dlb_status dlb_model_set_array(dlb_model *m, const char *name, const float *host_in, size_t n) {
  DLB_REQUIRE(m && name && host_in, "set_array: null");
  if (!m->params) DLB_TRY(allocate_parameters(m));
  float *p = named_array(m, name);
  DLB_REQUIRE(p && n <= m->total_parameters, "set_array: unknown name or size");
  if (p == m->m1 || p == m->m2 || p == m->m2hat) DLB_TRY(gather_moments(m));
  DLB_TRY(dlb_memcpy_h2d(m->ctx, p, host_in, n * sizeof(float)));
  DLB_TRY(dlb_ctx_sync(m->ctx, nullptr));
  if (p == m->params) m->params_lo_valid = false;
  if (p == m->grads) m->grads_clean = false;
  return DLB_OK;
}

static dlb_status layer_norm_io(dlb_model *m, size_t layer, const char *name, float *out,
                                const float *in, size_t n) {
  DLB_REQUIRE(m && name && layer_at(m, layer), "layer_norm: bad layer");
  LayerRT &l = m->layers[layer];
  DLB_REQUIRE(l.norm != DLB_NORM_NONE, "layer_norm: layer is not normalised");
  if (!m->params) DLB_TRY(allocate_parameters(m));
  DLB_TRY(ensure_norm_state(m));
  const std::string nm(name);
  float *dev = nullptr;
  size_t count = 0;
  if (nm == "scale") { dev = m->params + gamma_index(m, l); count = l.norm_units; }
  else if (nm == "shift") { dev = m->params + beta_index(m, l); count = l.norm_units; }
  else {
    const int f = norm_field(nm);
    DLB_REQUIRE(f >= 0, "layer_norm: unknown field");
    count = m->seq_w * l.norm_units;
    dev = l.stats + (size_t)f * count;
  }
  DLB_REQUIRE(n == count, "layer_norm: size mismatch");
  if (out) return dlb_memcpy_d2h(m->ctx, out, dev, n * sizeof(float));
  DLB_TRY(dlb_memcpy_h2d(m->ctx, dev, in, n * sizeof(float)));
  return dlb_ctx_sync(m->ctx, nullptr);
}

dlb_status dlb_model_get_layer_norm(dlb_model *m, size_t layer, const char *name, float *host_out,
                                    size_t n) {
  DLB_REQUIRE(host_out, "get_layer_norm: null");
  return layer_norm_io(m, layer, name, host_out, nullptr, n);
}
dlb_status dlb_model_set_layer_norm(dlb_model *m, size_t layer, const char *name,
                                    const float *host_in, size_t n) {
  DLB_REQUIRE(host_in, "set_layer_norm: null");
  return layer_norm_io(m, layer, name, nullptr, host_in, n);
}

dlb_status dlb_model_set_dropout_mask(dlb_model *m, size_t layer, const uint8_t *host_mask,
                                      size_t n) {
  DLB_REQUIRE(m && host_mask && layer_at(m, layer), "set_dropout_mask");
  LayerRT &l = m->layers[layer];
  DLB_REQUIRE(n == m->seq_w * l.units, "set_dropout_mask: size mismatch");
  DLB_TRY(ensure_masks(m));
  DLB_REQUIRE(l.mask, "set_dropout_mask: layer has no Bernoulli dropout");
  std::vector<uint8_t> norm01(n);
  for (size_t i = 0; i < n; ++i) norm01[i] = host_mask[i] ? 1 : 0;
  DLB_TRY(dlb_memcpy_h2d(m->ctx, l.mask, norm01.data(), n));
  return dlb_ctx_sync(m->ctx, nullptr);
}

// A block layer's dropout acts on its input (pre-activation order).
static size_t uout_width(const LayerRT &l) { return l.group == 1 ? l.fan_in : l.units; }

static dlb_status ensure_uout(dlb_model *m, LayerRT &l, size_t rows) {
  if (rows <= l.uout_rows) return DLB_OK;
  if (l.uout) DLB_TRY(dlb_free(m->ctx, l.uout));
  l.uout = nullptr;
  l.uout_rows = 0;
  DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.uout), rows * uout_width(l) * sizeof(float)));
  l.uout_rows = rows;
  return DLB_OK;
}

static dlb_status ensure_shakedrop(dlb_model *m, LayerRT &l, size_t rows) {
  if (rows <= l.sd_rows) return DLB_OK;
  if (l.sd_mask) DLB_TRY(dlb_free(m->ctx, l.sd_mask));
  if (l.sd_fwd) DLB_TRY(dlb_free(m->ctx, l.sd_fwd));
  if (l.sd_bwd) DLB_TRY(dlb_free(m->ctx, l.sd_bwd));
  l.sd_mask = nullptr;
  l.sd_fwd = l.sd_bwd = nullptr;
  l.sd_rows = 0;
  DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.sd_mask), rows));
  DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.sd_fwd), rows * l.norm_units * sizeof(float)));
  DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&l.sd_bwd), rows * l.norm_units * sizeof(float)));
  l.sd_rows = rows;
  return DLB_OK;
}

dlb_status dlb_model_set_uout_noise(dlb_model *m, size_t layer, const float *host_noise, size_t rows) {
  DLB_REQUIRE(m && host_noise && layer_at(m, layer) && rows > 0, "set_uout_noise");
  LayerRT &l = m->layers[layer];
  DLB_REQUIRE(l.dropout == DLB_DROPOUT_UOUT, "set_uout_noise: layer does not use UOut");
  DLB_TRY(ensure_uout(m, l, rows));
  DLB_TRY(dlb_memcpy_h2d(m->ctx, l.uout, host_noise, rows * uout_width(l) * sizeof(float)));
  return dlb_ctx_sync(m->ctx, nullptr);
}

// The step's noise drawn on the device (csrc/noise.cu) instead of handed over:
// per layer, stream 4 * layer + {0: Bernoulli flags, 1: forward draws, 2:
// backward draws}.  Masks of Bernoulli dropout have one flag per unit (every
// row shares it, Model::Dropout_Bernoulli); UOut and ShakeDrop arrays have one
// row per example and are indexed by the example's row in the whole batch,
// first_row + r, so that every sharding of the batch draws the same array.
dlb_status dlb_model_draw_noise(dlb_model *m, size_t rows, uint64_t seed, uint32_t step, size_t first_row) {
  DLB_REQUIRE(m && rows > 0, "draw_noise");
  DLB_TRY(check_supported(m));
  DLB_TRY(ensure_masks(m));
  for (size_t i = 0; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    const uint32_t stream = 4u * (uint32_t)i;
    switch (l.dropout) {
      case DLB_DROPOUT_BERNOULLI:
      case DLB_DROPOUT_BERNOULLI_INVERTED:
        // dropout_value is the probability that a unit is kept.
        DLB_TRY(dlb_noise_bernoulli(m->ctx, l.mask, m->seq_w * l.units, l.dropout_value, seed, stream, step, 0));
        break;
      case DLB_DROPOUT_UOUT: {
        const size_t w = uout_width(l);
        DLB_TRY(ensure_uout(m, l, rows));
        DLB_TRY(dlb_noise_uniform(m->ctx, l.uout, rows * w, -l.dropout_value, l.dropout_value, seed, stream + 1,
                                  step, first_row * w));
        break;
      }
      case DLB_DROPOUT_SHAKEDROP:
        // dropout_value is the probability that a row is perturbed; forward
        // factors from U(-1, 1), backward factors from U(0, 1)
        // (fwp_mp.cpp L:3881-3888, bwp_mp.cpp ShakeDrop backward).
        DLB_TRY(ensure_shakedrop(m, l, rows));
        DLB_TRY(dlb_noise_bernoulli(m->ctx, l.sd_mask, rows, l.dropout_value, seed, stream, step, first_row));
        // (one factor per element of the block's output, norm_units wide)
        DLB_TRY(dlb_noise_uniform(m->ctx, l.sd_fwd, rows * l.norm_units, -1.f, 1.f, seed, stream + 1, step,
                                  first_row * l.norm_units));
        DLB_TRY(dlb_noise_uniform(m->ctx, l.sd_bwd, rows * l.norm_units, 0.f, 1.f, seed, stream + 2, step,
                                  first_row * l.norm_units));
        break;
      default:
        break;
    }
  }
  return DLB_OK;
}

dlb_status dlb_model_set_shakedrop_noise(dlb_model *m, size_t layer, const uint8_t *host_row_mask,
                                         const float *host_forward, const float *host_backward,
                                         size_t rows) {
  DLB_REQUIRE(m && host_row_mask && host_forward && host_backward && layer_at(m, layer) && rows > 0,
              "set_shakedrop_noise");
  LayerRT &l = m->layers[layer];
  DLB_REQUIRE(l.type == DLB_LAYER_RESIDUAL && l.dropout == DLB_DROPOUT_SHAKEDROP,
              "set_shakedrop_noise: layer is not a residual layer with ShakeDrop");
  const size_t n = rows * l.norm_units;  // one factor per element of the block's output
  DLB_TRY(ensure_shakedrop(m, l, rows));
  std::vector<uint8_t> flags(rows);
  for (size_t i = 0; i < rows; ++i) flags[i] = host_row_mask[i] ? 1 : 0;
  DLB_TRY(dlb_memcpy_h2d(m->ctx, l.sd_mask, flags.data(), rows));
  DLB_TRY(dlb_memcpy_h2d(m->ctx, l.sd_fwd, host_forward, n * sizeof(float)));
  DLB_TRY(dlb_memcpy_h2d(m->ctx, l.sd_bwd, host_backward, n * sizeof(float)));
  return dlb_ctx_sync(m->ctx, nullptr);
}

dlb_status dlb_model_set_global_batch(dlb_model *m, size_t global_rows) {
  DLB_REQUIRE(m, "null");
  m->global_rows = global_rows;
  return DLB_OK;
}

// Number of examples of the training set, the `training_size` that the one-call
// steps pass to update_weights (Model::normalized_wd divides the batch size by
// it, v1/learner/train.cpp L:278-283).  0 (default): one batch is the whole set.
dlb_status dlb_model_set_training_size(dlb_model *m, size_t training_size) {
  DLB_REQUIRE(m, "null");
  m->training_size = training_size;
  return DLB_OK;
}

dlb_status dlb_model_forward_pass_device(dlb_model *m, size_t rows, const float *X_dev) {
  DLB_REQUIRE(m && X_dev && rows > 0, "forward_pass_device");
  DLB_TRY(check_supported(m));
  DLB_TRY(ensure_batch(m, rows));
  const size_t n = rows * m->seq_w * n_in(m);
  if (time_stepped(m)) {
    // [rows, T * n_in] -> [T, rows, n_in] with the residual plane in the same pass.
    DLB_REQUIRE(X_dev != m->input, "forward_pass_device: input aliases the model's own buffer");
    DLB_REQUIRE(rows * m->seq_w < ((size_t)1 << 31), "forward_pass_device: rows * seq_w overflows int");
    DLB_TRY(dlb_time_major(m->ctx, X_dev, m->input, m->input_lo, (int)rows, (int)m->seq_w, (int)n_in(m)));
    // Dropout on the inputs, per time step and unit, on the model's copy of the
    // batch (Model::assign_inputs_rec_mp, v1/learner/assign_inputs.cpp L:219-266):
    // the Bernoulli kinds by the input layer's mask in training, the plain kind by
    // its keep probability at inference.  One walk in place (no recurrence, no
    // activation), which also writes the planes of the masked batch.
    const LayerRT &in0 = m->layers[0];
    const bool bern0 = in0.dropout == DLB_DROPOUT_BERNOULLI || in0.dropout == DLB_DROPOUT_BERNOULLI_INVERTED;
    if (bern0 && m->propagation == DLB_PROPAGATION_TRAINING) {
      const float keep_scale = in0.dropout == DLB_DROPOUT_BERNOULLI_INVERTED
                                   ? (in0.dropout_value == 0.f ? 0.f : 1.f / in0.dropout_value)
                                   : 1.f;
      DLB_TRY(dlb_indrnn_forward_dropout(m->ctx, m->input, nullptr, nullptr, DLB_AF_LINEAR, in0.mask, keep_scale,
                                         m->input, m->input_lo, (int)m->seq_w, (int)rows, (int)n_in(m)));
    } else if (in0.dropout == DLB_DROPOUT_BERNOULLI) {
      DLB_TRY(dlb_indrnn_forward_dropout(m->ctx, m->input, nullptr, nullptr, DLB_AF_LINEAR, nullptr, in0.dropout_value,
                                         m->input, m->input_lo, (int)m->seq_w, (int)rows, (int)n_in(m)));
    }
    return forward_layers(m, rows);
  }
  if (X_dev != m->input) DLB_TRY(dlb_memcpy_d2d(m->ctx, m->input, X_dev, n * sizeof(float)));
  // Dropout on the inputs acts on the model's copy of the batch, in place
  // (Model::assign_inputs_fwp_mp, v1/learner/assign_inputs.cpp L:94-130): the
  // Bernoulli kinds by the input layer's mask in training, the plain kind by its
  // keep probability at inference.
  const LayerRT &in = m->layers[0];
  const bool bern = in.dropout == DLB_DROPOUT_BERNOULLI || in.dropout == DLB_DROPOUT_BERNOULLI_INVERTED;
  if (bern && m->propagation == DLB_PROPAGATION_TRAINING) {
    dlb_dropout_desc dp{in.dropout, in.dropout_value, in.mask, nullptr};
    DLB_TRY(dlb_activation_forward(m->ctx, m->input, nullptr, DLB_AF_LINEAR, &dp, m->input, m->input_lo,
                                   (int)rows, (int)n_in(m)));
  } else if (in.dropout == DLB_DROPOUT_BERNOULLI) {
    dlb_dropout_desc dp{DROPOUT_INFERENCE_SCALE, in.dropout_value, nullptr, nullptr};
    DLB_TRY(dlb_activation_forward(m->ctx, m->input, nullptr, DLB_AF_LINEAR, &dp, m->input, m->input_lo,
                                   (int)rows, (int)n_in(m)));
  } else {
    DLB_TRY(dlb_split_planes_2d(m->ctx, m->input, m->input_lo, (int)rows, (int)n_in(m)));
  }
  return forward_layers(m, rows);
}

dlb_status dlb_model_forward_pass(dlb_model *m, size_t rows, const float *const *Xm) {
  DLB_REQUIRE(m && Xm && rows > 0, "forward_pass");
  DLB_TRY(check_supported(m));
  DLB_TRY(ensure_batch(m, rows));
  float *dst = time_stepped(m) ? m->input_rows : m->input;
  DLB_TRY(stage_rows(m, 0, &m->stage_x, &m->stage_x_elems, rows, m->seq_w * n_in(m), Xm, dst));
  DLB_TRY(dlb_model_forward_pass_device(m, rows, dst));
  return rows_consumed(m, 0);
}

dlb_status dlb_model_compute_error_device(dlb_model *m, size_t rows, const float *Y_dev) {
  DLB_REQUIRE(m && Y_dev && rows > 0 && rows <= m->alloc_rows, "compute_error_device");
  LayerRT &o = m->layers.back();
  const int Bg = (int)(m->global_rows ? m->global_rows : rows);
  if (time_stepped(m)) {
    // The error exists for t >= n_time_delay only, each step with the divisor
    // of one batch; earlier steps carry a zero error
    // (compute_error_rec_mp, v1/learner/compute_error_mp.cpp L:143-265).
    DLB_REQUIRE(Y_dev != m->target, "compute_error_device: target aliases the model's own buffer");
    const size_t T = m->seq_w, d = m->n_time_delay, W = o.units;
    DLB_TRY(dlb_time_major(m->ctx, Y_dev, m->target, nullptr, (int)rows, (int)T, (int)W));
    const size_t skip = d * rows * W;
    if (skip) {
      DLB_TRY(dlb_memset(m->ctx, o.delta, 0, skip * sizeof(float)));
      DLB_TRY(dlb_memset(m->ctx, o.delta_lo, 0, skip * sizeof(float)));
    }
    DLB_TRY(dlb_loss_delta(m->ctx, m->loss, o.af, o.Z + skip, o.A + skip, m->target + skip,
                           o.delta + skip, o.delta_lo + skip, (int)((T - d) * rows), (int)W, Bg,
                           m->loss_sum));
    if (o.af == DLB_AF_SOFTMAX && T > 1) {
      // The softmax branch of compute_error_rec_mp takes the error of every time
      // step against the target of time step 0 (`Ym[i][k]`,
      // v1/learner/compute_error_mp.cpp L:237-247) while the loss above reads the
      // step's own target: the error is formed again against time step 0's rows.
      const size_t block = rows * W;
      void *scr = nullptr;
      DLB_TRY(scratch(m->ctx, (T - d) * block * sizeof(float) + 256, &scr));
      float *first = static_cast<float *>(scr);
      double *unused = reinterpret_cast<double *>(first + align_up((T - d) * block, 64));
      for (size_t t = 0; t < T - d; ++t)
        DLB_TRY(dlb_memcpy_d2d(m->ctx, first + t * block, m->target, block * sizeof(float)));
      DLB_TRY(dlb_loss_delta(m->ctx, m->loss, o.af, o.Z + skip, o.A + skip, first, o.delta + skip,
                             o.delta_lo + skip, (int)((T - d) * rows), (int)W, Bg, unused));
    }
    // The accuracy counter of the training pass (compute_error_rec_mp,
    // v1/learner/compute_error_mp.cpp L:178-231), when asked for.
    if (m->training_accuracy)
      DLB_TRY(dlb_loss_eval(m->ctx, m->loss, m->accu_fn, m->accu_var, o.A + skip, m->target + skip,
                            (int)((T - d) * rows), (int)W, nullptr, m->accu_sum));
    m->loss_rows += rows * (T - d);
    return DLB_OK;
  }
  DLB_TRY(dlb_loss_delta(m->ctx, m->loss, o.af, o.Z, o.A, Y_dev, o.delta, o.delta_lo, (int)rows,
                         (int)o.units, Bg, m->loss_sum));
  // compute_error_fwp_mp counts the accuracy as well (compute_error_mp.cpp L:60-112).
  if (m->training_accuracy)
    DLB_TRY(dlb_loss_eval(m->ctx, m->loss, m->accu_fn, m->accu_var, o.A, Y_dev, (int)rows, (int)o.units, nullptr,
                          m->accu_sum));
  m->loss_rows += rows;
  return DLB_OK;
}

dlb_status dlb_model_compute_error(dlb_model *m, size_t rows, const float *const *Ym) {
  DLB_REQUIRE(m && Ym && rows > 0 && rows <= m->alloc_rows, "compute_error");
  float *dst = time_stepped(m) ? m->target_rows : m->target;
  DLB_TRY(stage_rows(m, 1, &m->stage_y, &m->stage_y_elems, rows, m->seq_w * n_out(m), Ym, dst));
  DLB_TRY(dlb_model_compute_error_device(m, rows, dst));
  return rows_consumed(m, 1);
}

static std::vector<size_t> top_level(const dlb_model *m) {
  std::vector<size_t> t;
  for (size_t i = 0; i < m->layers.size(); ++i)
    if (m->layers[i].group == 0) t.push_back(i);
  return t;
}

// ref: Backward_Pass__Residual__Block__OpenMP and
// Backward_Pass__Gradient__Residual__FC__OpenMP (v1/learner/bwp_mp.cpp
// L:310-406, L:658-874): the error of the residual output becomes the error of
// the block output (ShakeDrop rows scaled by fresh U(0,1), then the residual
// layer's normalization), then the block layers from last to first.
static dlb_status backward_residual(dlb_model *m, size_t i, int B) {
  LayerRT &res = m->layers[i];
  LayerRT &last = m->layers[i + res.depth];
  const bool shake = res.dropout == DLB_DROPOUT_SHAKEDROP;
  const bool rnorm = res.norm != DLB_NORM_NONE;
  // The block reads its window of the residual layer's error.
  const int first = last.units < res.units ? (int)res.pad : 0;
  DLB_TRY(dlb_shakedrop_backward_window(m->ctx, res.delta, (int)res.units, first, shake ? res.sd_mask : nullptr,
                                        shake ? res.sd_bwd : nullptr, last.delta,
                                        rnorm ? nullptr : last.delta_lo, B, (int)last.units));
  if (rnorm)
    DLB_TRY(norm_backward(m, res, last.delta, last.delta_lo, last.A, last.A, DLB_AF_LINEAR, B));
  for (size_t j = res.depth; j >= 2; --j) {
    LayerRT &b = m->layers[i + j];
    LayerRT &prev = m->layers[i + j - 1];
    DLB_TRY(dlb_fc_backward_input(m->ctx, b.delta, b.delta_lo, m->params + b.first_conn,
                                  m->params_lo + b.first_conn, prev.delta, B, (int)b.fan_in,
                                  (int)b.units));
    if (b.norm != DLB_NORM_NONE) {
      DLB_TRY(norm_backward(m, b, prev.delta, prev.delta_lo, prev.A, b.IN, b.af, B));
    } else {
      DLB_TRY(dlb_activation_backward(m->ctx, prev.delta, prev.A, b.IN, nullptr, b.af, B,
                                      (int)b.fan_in, nullptr));
      DLB_TRY(dlb_split_planes_2d(m->ctx, prev.delta, prev.delta_lo, B, (int)b.fan_in));
    }
  }
  return DLB_OK;
}

// Backward of a residual block inside a time-stepped model: backward_residual
// over the T * B rows with the per-time-step normalization backward.
static dlb_status backward_residual_time(dlb_model *m, size_t i, int B, int T) {
  LayerRT &res = m->layers[i];
  LayerRT &last = m->layers[i + res.depth];
  const int TB = T * B;
  const bool shake = res.dropout == DLB_DROPOUT_SHAKEDROP;
  const bool rnorm = res.norm != DLB_NORM_NONE;
  const int first = last.units < res.units ? (int)res.pad : 0;
  DLB_TRY(dlb_shakedrop_backward_window(m->ctx, res.delta, (int)res.units, first, shake ? res.sd_mask : nullptr,
                                        shake ? res.sd_bwd : nullptr, last.delta,
                                        rnorm ? nullptr : last.delta_lo, TB, (int)last.units));
  if (rnorm) DLB_TRY(norm_backward_time(m, res, last.delta, last.delta_lo, last.A, last.A, DLB_AF_LINEAR, T, B));
  for (size_t j = res.depth; j >= 2; --j) {
    LayerRT &b = m->layers[i + j];
    LayerRT &prev = m->layers[i + j - 1];
    DLB_TRY(dlb_fc_backward_input(m->ctx, b.delta, b.delta_lo, m->params + b.first_conn, m->params_lo + b.first_conn,
                                  prev.delta, TB, (int)b.fan_in, (int)b.units));
    if (b.norm != DLB_NORM_NONE) {
      DLB_TRY(norm_backward_time(m, b, prev.delta, prev.delta_lo, prev.A, b.IN, b.af, T, B));
    } else {
      DLB_TRY(dlb_activation_backward(m->ctx, prev.delta, prev.A, b.IN, nullptr, b.af, TB, (int)b.fan_in, nullptr));
      DLB_TRY(dlb_split_planes_2d(m->ctx, prev.delta, prev.delta_lo, TB, (int)b.fan_in));
    }
  }
  return DLB_OK;
}

// ref: Model::RNN__Backward_Pass_Batch__OpenMP (v1/learner/bwp_rec_mp.cpp
// L:29-110) with Backward_Pass__FC__DF_Ind_RNN__OpenMP (bwp_mp.cpp L:1188-1263)
// and the recurrent-weight gradient of update_derivative_rec_mp.cpp L:460-487,
// which is formed here because it shares its pass over dAF with the
// batch-renormalization sums.
static dlb_status backward_pass_time(dlb_model *m, size_t rows) {
  const int B = (int)rows, T = (int)m->seq_w;
  const int TB = T * B;
  const int Bg = (int)(m->global_rows ? m->global_rows : rows);
  const std::vector<size_t> tops = top_level(m);
  for (size_t pos = tops.size() - 1; pos >= 1; --pos) {
    const size_t i = tops[pos];
    LayerRT &l = m->layers[i];
    LayerRT *below = pos > 1 ? &m->layers[tops[pos - 1]] : nullptr;  // the error into the input layer is never formed
    if (l.type == DLB_LAYER_RESIDUAL) {
      DLB_TRY(backward_residual_time(m, i, B, T));
      if (below) {
        // shortcut error (its window of the residual layer's error) + delta_1 W_1
        LayerRT &first = m->layers[i + 1];
        const size_t first_col = l.fan_in < l.units ? l.pad : 0;
        DLB_CUDA(cudaMemcpy2DAsync(below->delta, l.fan_in * sizeof(float), l.delta + first_col,
                                   l.units * sizeof(float), l.fan_in * sizeof(float), (size_t)TB,
                                   cudaMemcpyDeviceToDevice, m->ctx->stream));
        GemmOperand A{first.delta, first.delta_lo, (long long)first.units, 1};
        GemmOperand Bo{m->params + first.first_conn, m->params_lo + first.first_conn, 1, (long long)first.fan_in};
        GemmEpilogue ep;
        ep.accumulate = 1;
        DLB_TRY(gemm(m->ctx, A, Bo, below->delta, (long long)first.fan_in, TB, (int)first.fan_in, (int)first.units, ep));
      }
      continue;
    }
    if (is_lstm(l)) {
      DLB_TRY(backward_lstm(m, l, below ? below->delta : nullptr, B, T));
      continue;
    }
    const int H = (int)l.units;
    const bool norm = l.norm != DLB_NORM_NONE, rec = is_indrnn(l);
    // Rows of this layer's error that can be non-zero.
    size_t first_row = 0;
    if (pos + 1 == tops.size()) {
      first_row = m->n_time_delay * rows;
    } else if (norm || rec) {  // hidden layer: l.delta holds dA
      const float *u_rec = rec ? m->params + l.first_recurrent : nullptr;
      dlb_brn_unit_arrays u{};
      if (norm) u = unit_arrays(m, l, 0);
      DLB_TRY(dlb_indrnn_backward_walk(m->ctx, l.delta, l.Z, l.A, norm ? &u : nullptr, u_rec, l.af, T, B, H));
      DLB_TRY(dlb_indrnn_backward_sums(m->ctx, l.delta, l.Z, l.A, norm ? &u : nullptr, rec ? 1 : 0, T, B,
                                       H, l.bwd_sums));
      const size_t plane = (size_t)T * H;
      if (rec)
        DLB_TRY(dlb_time_fold(m->ctx, l.bwd_sums + (norm ? 4 : 0) * plane, T, H,
                              m->grads + l.first_recurrent));
      if (norm) {
        DLB_TRY(dlb_time_fold(m->ctx, l.bwd_sums, T, H, m->grads + gamma_index(m, l)));
        DLB_TRY(dlb_time_fold(m->ctx, l.bwd_sums + plane, T, H, m->grads + beta_index(m, l)));
        DLB_TRY(dlb_allreduce_f64(m->ctx, l.bwd_sums + 2 * plane, 2 * plane));
        DLB_TRY(dlb_brn_time_backward_apply(m->ctx, l.delta, l.delta_lo, l.Z, &u, l.bwd_sums, Bg, T, B, H));
      } else {
        DLB_TRY(dlb_split_planes_2d(m->ctx, l.delta, l.delta_lo, TB, H));
      }
    } else {
      DLB_TRY(dlb_activation_backward(m->ctx, l.delta, l.Z, l.A, nullptr, l.af, TB, H, nullptr));
      DLB_TRY(dlb_split_planes_2d(m->ctx, l.delta, l.delta_lo, TB, H));
    }
    if (!below) break;
    const size_t I = l.fan_in;
    if (first_row) DLB_TRY(dlb_memset(m->ctx, below->delta, 0, first_row * I * sizeof(float)));
    if (first_row < (size_t)TB)
      DLB_TRY(dlb_fc_backward_input(m->ctx, l.delta + first_row * H, l.delta_lo + first_row * H,
                                    m->params + l.first_conn, m->params_lo + l.first_conn,
                                    below->delta + first_row * I, TB - (int)first_row, (int)I, H));
  }
  return DLB_OK;
}

// ref: Model::FF__Backward_Pass_Batch__OpenMP (v1/learner/bwp_mp.cpp L:28-208):
// from the output layer down; the error into the input layer is never formed.
dlb_status dlb_model_backward_pass(dlb_model *m, size_t rows) {
  DLB_REQUIRE(m && rows > 0 && rows <= m->alloc_rows, "backward_pass");
  if (time_stepped(m)) return backward_pass_time(m, rows);
  const int B = (int)rows;
  const std::vector<size_t> tops = top_level(m);
  for (size_t pos = tops.size() - 1; pos >= 1; --pos) {
    const size_t i = tops[pos];
    LayerRT &l = m->layers[i];
    LayerRT *below = pos > 1 ? &m->layers[tops[pos - 1]] : nullptr;
    if (l.type == DLB_LAYER_RESIDUAL) {
      DLB_TRY(backward_residual(m, i, B));
      if (below) {
        // shortcut error + delta_1 W_1
        LayerRT &first = m->layers[i + 1];
        // (the shortcut's window of the residual layer's error)
        const size_t first_col = l.fan_in < l.units ? l.pad : 0;
        DLB_CUDA(cudaMemcpy2DAsync(below->delta, l.fan_in * sizeof(float), l.delta + first_col,
                                   l.units * sizeof(float), l.fan_in * sizeof(float), (size_t)B,
                                   cudaMemcpyDeviceToDevice, m->ctx->stream));
        GemmOperand A{first.delta, first.delta_lo, (long long)first.units, 1};
        GemmOperand Bo{m->params + first.first_conn, m->params_lo + first.first_conn, 1,
                       (long long)first.fan_in};
        GemmEpilogue ep;
        ep.accumulate = 1;
        DLB_TRY(gemm(m->ctx, A, Bo, below->delta, (long long)first.fan_in, B, (int)first.fan_in,
                     (int)first.units, ep));
      }
      continue;
    }
    const int H = (int)l.units;
    if (pos + 1 != tops.size() && !l.error_final) {  // hidden layer: l.delta holds dA
      if (l.norm != DLB_NORM_NONE) {
        DLB_TRY(norm_backward(m, l, l.delta, l.delta_lo, l.Z, l.A, l.af, B));
      } else {
        DLB_TRY(dlb_activation_backward(m->ctx, l.delta, l.Z, l.A, nullptr, l.af, B, H, nullptr));
        DLB_TRY(dlb_split_planes_2d(m->ctx, l.delta, l.delta_lo, B, H));
      }
    }
    l.error_final = false;
    if (below) {
      if (below->type != DLB_LAYER_RESIDUAL && below->norm == DLB_NORM_NONE && pos > 1) {
        // The layer below has no normalization: its activation derivative rides
        // in this product's epilogue and below->delta is its final error.
        DLB_TRY(dlb_fc_backward_input_derivative(m->ctx, l.delta, l.delta_lo, m->params + l.first_conn,
                                                 m->params_lo + l.first_conn, below->Z, below->A, below->af,
                                                 below->delta, below->delta_lo, B, (int)l.fan_in, H));
        below->error_final = true;
      } else {
        DLB_TRY(dlb_fc_backward_input(m->ctx, l.delta, l.delta_lo, m->params + l.first_conn,
                                      m->params_lo + l.first_conn, below->delta, B, (int)l.fan_in, H));
      }
    }
  }
  return DLB_OK;
}

// ref: Model::RNN__Update_Derivative_Weight_Batch__OpenMP
// (v1/learner/update_derivative_rec_mp.cpp L:27-167): the per-time-step rank-1
// sums of a layer are one GEMM whose reduction runs over all T * rows rows.
static dlb_status prepare_update(dlb_model *m, size_t rows, size_t training_size, dlb_optimizer_scalars *out);
static dlb_status update_segment(dlb_model *m, const dlb_optimizer_scalars &k, size_t at, size_t n, unsigned *amax);

// Owner-computes update of the weight matrices across ranks, inside a one-call
// step (see backward_and_derivatives_overlapped).  Every weight matrix must
// divide by rows among the ranks and the weights must be fully connected
// matrices only (no recurrent weights between them).
static bool sharded_update_possible(const dlb_model *m) {
  static const bool off = getenv("DLB_SHARDED_UPDATE") && atoi(getenv("DLB_SHARDED_UPDATE")) == 0;
  if (off || !m->sharded_update || !comm_can_shard(m->ctx) || m->use_clip_gradient || !m->optimizer) return false;
  if (m->ctx->gemm_kind != DLB_GEMM_F16X3 || !m->params_lo || time_stepped(m)) return false;
  const size_t W = (size_t)dlb_comm_world(m->ctx);
  size_t weights = 0;
  for (size_t i = 1; i < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;
    if (l.type != DLB_LAYER_FULLY_CONNECTED || l.last_conn - l.first_conn != l.units * l.fan_in) return false;
    if (l.units % W != 0 || ((l.first_conn | (l.units / W * l.fan_in)) & 3) != 0) return false;
    weights += l.units * l.fan_in;
  }
  return weights == m->total_weights;
}

// One step's owner-computes updates.  begin() draws the step's scalars;
// reduce(l) follows the layer's weight-gradient product; update(l) comes once
// no product of the step reads the layer's weights any more; finish() before
// the streams are joined.  The planes of a gathered matrix are formed one call
// later, when its gather has had time.
struct OwnerUpdate {
  dlb_model *m;
  size_t W, rank;
  LayerRT *to_split = nullptr;
  explicit OwnerUpdate(dlb_model *model)
      : m(model), W((size_t)dlb_comm_world(model->ctx)), rank((size_t)dlb_comm_rank(model->ctx)) {}
  size_t per(const LayerRT &l) const { return l.units / W * l.fan_in; }
  dlb_status begin(size_t update_rows, size_t training_size) {
    DLB_TRY(prepare_update(m, update_rows, training_size, &m->update_k));
    m->update_prepared = true;
    m->moments_sharded = true;
    return DLB_OK;
  }
  dlb_status split_gathered() {
    if (!to_split) return DLB_OK;
    LayerRT &g = *to_split;
    to_split = nullptr;
    DLB_TRY(comm_wait(m->ctx, g.ev_gathered));
    return dlb_split_planes_2d(m->ctx, m->params + g.first_conn, m->params_lo + g.first_conn, (int)g.units,
                               (int)g.fan_in);
  }
  dlb_status reduce(LayerRT &l) {
    DLB_TRY(comm_reduce_scatter_begin(m->ctx, m->grads + l.first_conn, per(l), &l.ev_reduced));
    return split_gathered();
  }
  dlb_status update(LayerRT &l) {
    DLB_TRY(comm_wait(m->ctx, l.ev_reduced));
    DLB_TRY(update_segment(m, m->update_k, l.first_conn + rank * per(l), per(l), nullptr));
    DLB_TRY(comm_all_gather_begin(m->ctx, m->params + l.first_conn, per(l), m->grads + l.first_conn, &l.ev_gathered));
    to_split = &l;
    return DLB_OK;
  }
  // After the backward pass, where nothing reads the weights any more: the
  // update of a layer follows the weight-gradient product of the next one, so
  // that its reduce-scatter has that product's time.
  LayerRT *pending = nullptr;
  dlb_status after_gradient(LayerRT &l) {
    DLB_TRY(reduce(l));
    if (pending) DLB_TRY(update(*pending));
    pending = &l;
    return DLB_OK;
  }
  dlb_status finish() {
    if (pending) {
      DLB_TRY(split_gathered());
      DLB_TRY(update(*pending));
      pending = nullptr;
    }
    return split_gathered();
  }
};

static dlb_status update_derivatives_time(dlb_model *m, size_t rows) {
  const size_t TB = m->seq_w * rows;
  const float *top = m->input, *top_lo = m->input_lo;  // output of the top-level layer below
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;  // its block layers follow; its output is set after them
    const float *X = top, *X_lo = top_lo;
    if (l.group == 1 && !l.block_input) {
      X = l.IN;
      X_lo = l.IN_lo;
    }
    if (is_lstm(l)) {
      DLB_TRY(derivatives_lstm(m, l, X, X_lo, (int)rows, (int)m->seq_w));
      if (m->overlap_grad_allreduce)
        DLB_TRY(dlb_allreduce_f32_overlapped(m->ctx, m->grads + l.first_conn, l.last_conn - l.first_conn));
      top = l.A;
      top_lo = l.A_lo;
      continue;
    }
    const size_t H = l.units, I = l.fan_in;
    // The output layer's error is zero before the first step that has a target.
    const size_t first_row = i + 1 == m->layers.size() ? m->n_time_delay * rows : 0;
    float *dbias = l.norm == DLB_NORM_NONE ? m->grads + l.first_bias : nullptr;
    DLB_TRY(dlb_fc_weight_gradient(m->ctx, l.delta + first_row * H, l.delta_lo + first_row * H,
                                   X + first_row * I, X_lo + first_row * I, m->grads + l.first_conn,
                                   dbias, (int)(TB - first_row), (int)I, (int)H, m->grads_clean ? 0 : 1));
    if (m->overlap_grad_allreduce)
      DLB_TRY(dlb_allreduce_f32_overlapped(m->ctx, m->grads + l.first_conn, l.last_conn - l.first_conn));
    if (l.group == 0) {
      top = l.A;
      top_lo = l.A_lo;
    } else if (i + 1 < m->layers.size() && m->layers[i + 1].group == 0) {
      // last layer of a block: what follows reads the residual layer's output
      size_t r = i;
      while (m->layers[r].type != DLB_LAYER_RESIDUAL) --r;
      top = m->layers[r].A;
      top_lo = m->layers[r].A_lo;
    }
  }
  // LSTM bias gradients last: they are added at the reference's indices, part of
  // which the next layer's bias gradient has just written.
  for (LayerRT &l : m->layers)
    if (is_lstm(l))
      DLB_TRY(dlb_scatter_add_rows(m->ctx, l.lstm_dbias, l.lstm_map_bias, m->grads, lstm_gates(l), 1));
  m->grads_clean = false;
  return DLB_OK;
}

// ref: Model::update_derivatives (v1/learner/update_derivative_fwp_mp.cpp L:27-240).
static dlb_status update_derivatives_flat(dlb_model *m, size_t rows, OwnerUpdate *owners);

dlb_status dlb_model_update_derivatives(dlb_model *m, size_t rows) {
  DLB_REQUIRE(m && rows > 0 && rows <= m->alloc_rows, "update_derivatives");
  if (time_stepped(m)) return update_derivatives_time(m, rows);
  return update_derivatives_flat(m, rows, nullptr);
}

// owners: the step's owner-computes updates (one-call steps on several ranks), or null.
static dlb_status update_derivatives_flat(dlb_model *m, size_t rows, OwnerUpdate *owners) {
  const float *top = m->input, *top_lo = m->input_lo;  // output of the top-level layer below
  for (size_t i = 1; i < m->layers.size(); ++i) {
    LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;  // its block layers follow; its output is set after them
    const float *X = top, *X_lo = top_lo;
    if (l.group == 1 && !l.block_input) {
      X = l.IN;
      X_lo = l.IN_lo;
    }
    float *dbias = l.norm == DLB_NORM_NONE ? m->grads + l.first_bias : nullptr;
    DLB_TRY(fc_weight_gradient_lines(m->ctx, l.delta, l.delta_lo, X, X_lo, m->grads + l.first_conn, dbias,
                                     (int)rows, (int)l.fan_in, (int)l.units, m->grads_clean ? 0 : 1,
                                     class_error(m, i)));
    if (owners) {
      // The backward pass is over: nothing reads the weights any more.
      DLB_TRY(owners->after_gradient(l));
    } else if (m->overlap_grad_allreduce) {
      DLB_TRY(dlb_allreduce_f32_overlapped(m->ctx, m->grads + l.first_conn, l.last_conn - l.first_conn));
    }
    if (l.group == 0) {
      top = l.A;
      top_lo = l.A_lo;
    } else if (i + 1 < m->layers.size() && m->layers[i + 1].group == 0) {
      // last layer of a block: what follows reads the residual layer's output
      size_t r = i;
      while (m->layers[r].type != DLB_LAYER_RESIDUAL) --r;
      top = m->layers[r].A;
      top_lo = m->layers[r].A_lo;
    }
  }
  m->grads_clean = false;
  if (owners) DLB_TRY(owners->finish());
  return DLB_OK;
}

dlb_status dlb_model_merge_derivatives(dlb_model *m) {
  DLB_REQUIRE(m && m->grads, "merge_derivatives");
  if (m->overlap_grad_allreduce) {
    // The weight blocks are already in flight; bias, gamma and beta follow.
    DLB_TRY(dlb_allreduce_f32_overlapped(m->ctx, m->grads + m->total_weights,
                                         m->total_parameters - m->total_weights));
    return dlb_comm_join(m->ctx);
  }
  return dlb_allreduce_f32(m->ctx, m->grads, m->total_parameters);
}

// The scalars of one update: hyper-parameters, the advanced time step, the
// step's weight decay (and its mask, on first use).
static dlb_status prepare_update(dlb_model *m, size_t rows, size_t training_size, dlb_optimizer_scalars *out) {
  DLB_REQUIRE(m && m->params && rows > 0 && training_size > 0, "update_weights");
  if (!m->optimizer) {
    set_error("update_weights: no optimizer set");
    return DLB_ERR_INVALID;
  }
  // Decoupled weight decay: step += mask * wd * p with the normalised wd of
  // Model::normalized_wd (v1/learner/train.cpp L:278-283; the reference's default
  // use_normalized_weight_decay = true) and the mask of
  // Indexing_Regularization_Parameters (v1/learner/indexing.cpp L:58-81): 1 on
  // the weights, 0 on biases, scales and shifts.
  float wd = 0.f;
  if (m->hp.weight_decay != 0.f) {
    if (!m->wd_mask) {
      std::vector<float> mask(m->total_parameters, 0.f);
      for (size_t i = 0; i < m->total_weights; ++i) mask[i] = 1.f;
      DLB_TRY(dev_alloc(m, &m->wd_mask, m->total_parameters, false));
      DLB_TRY(dlb_memcpy_h2d(m->ctx, m->wd_mask, mask.data(), mask.size() * sizeof(float)));
      DLB_TRY(dlb_ctx_sync(m->ctx, nullptr));
    }
    wd = m->hp.use_normalized_weight_decay
             ? m->hp.weight_decay * sqrtf((float)rows / ((float)training_size * m->hp.epoch_time_step))
             : m->hp.weight_decay;
  }
  float hyper[8] = {m->hp.adam_learning_rate, m->hp.adam_beta1, m->hp.adam_beta2,
                    m->hp.adam_epsilon, m->hp.adam_gamma, m->hp.learning_rate_final,
                    m->hp.learning_gamma, m->hp.use_adam_bias_correction ? 1.f : 0.f};
  if (m->optimizer == DLB_OPT_GD) {
    hyper[0] = m->hp.learning_rate;
    hyper[1] = m->hp.learning_momentum;
    hyper[2] = m->hp.use_nesterov ? 1.f : 0.f;
  }
  DLB_TRY(dlb_optimizer_prepare(m->optimizer, hyper, &m->hp.optimizer_time_step,
                                &m->hp.adam_previous_beta2, out));
  out->weight_decay = wd;
  return DLB_OK;
}

// Moments of the weight matrices back on every rank after owner-computes
// updates.  A collective: every rank calls it at the same point.
static dlb_status gather_moments(dlb_model *m) {
  if (!m->moments_sharded) return DLB_OK;
  const size_t W = (size_t)dlb_comm_world(m->ctx);
  for (size_t i = 1; i < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    if (l.type == DLB_LAYER_RESIDUAL) continue;
    const size_t per = l.units * l.fan_in / W;
    for (float *v : {m->m1, m->m2, m->m2hat})
      if (v) DLB_TRY(comm_all_gather(m->ctx, v + l.first_conn, per));
  }
  m->moments_sharded = false;
  return DLB_OK;
}

// One rank's share of the update of a weight segment (same arithmetic per
// element as the whole-vector pass).
static dlb_status update_segment(dlb_model *m, const dlb_optimizer_scalars &k, size_t at, size_t n, unsigned *amax) {
  if (n == 0) return DLB_OK;
  return optimizer_step_amax(m->ctx, m->optimizer, &k, m->params + at, m->grads + at, m->m1 + at, m->m2 + at,
                             m->m2hat ? m->m2hat + at : nullptr, k.weight_decay != 0.f ? m->wd_mask + at : nullptr,
                             n, amax);
}

// ref: Model::update_weights_mp (v1/learner/model.cpp L:4711-4796).
dlb_status dlb_model_update_weights(dlb_model *m, size_t rows, size_t training_size) {
  DLB_REQUIRE(m && m->params && rows > 0 && training_size > 0, "update_weights");
  if (m->update_prepared) {
    // The step's backward pass has updated the weight matrices slice by slice
    // and split them; biases, scales and shifts follow here.
    m->update_prepared = false;
    DLB_TRY(update_segment(m, m->update_k, m->total_weights, m->total_parameters - m->total_weights, nullptr));
    m->grads_clean = true;
    m->params_lo_valid = true;
    return DLB_OK;
  }
  DLB_TRY(gather_moments(m));
  dlb_optimizer_scalars k;
  DLB_TRY(prepare_update(m, rows, training_size, &k));
  const float wd = k.weight_decay;
  if (m->use_clip_gradient)
    DLB_TRY(dlb_clip_gradient(m->ctx, m->grads, m->total_parameters, m->clip_gradient));
  // One pass per weight matrix where the products run on fp16 planes: the pass
  // leaves the matrix's largest |w| in the scale slot of its plane buffer and
  // the split follows at once, while the matrix is still partly in L2; the
  // next forward pass then finds the planes ready.  Everything between and
  // after the matrices (recurrent weights, biases, scales, shifts) goes in
  // passes of its own.
  bool fused = m->ctx->gemm_kind == DLB_GEMM_F16X3 && m->params_lo != nullptr;
  for (size_t i = 1; fused && i < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    if (l.type != DLB_LAYER_RESIDUAL && ((l.first_conn | (l.units * l.fan_in) | l.last_conn) & 3)) fused = false;
  }
  auto segment = [&](size_t at, size_t n, unsigned *amax) -> dlb_status {
    if (n == 0) return DLB_OK;
    return optimizer_step_amax(m->ctx, m->optimizer, &k, m->params + at, m->grads + at, m->m1 + at, m->m2 + at,
                               m->m2hat ? m->m2hat + at : nullptr, wd != 0.f ? m->wd_mask + at : nullptr, n, amax);
  };
  if (fused) {
    size_t at = 0;
    for (size_t i = 1; i < m->layers.size(); ++i) {
      const LayerRT &l = m->layers[i];
      if (l.type == DLB_LAYER_RESIDUAL) continue;
      const size_t nw = l.units * l.fan_in;
      DLB_TRY(segment(at, l.first_conn - at, nullptr));
      PlaneJob job;
      DLB_TRY(planes_open(m->ctx, m->params + l.first_conn, m->params_lo + l.first_conn, nw, (int)l.units,
                          (int)l.fan_in, true, &job));
      if (job.fused) {
        const size_t o = l.first_conn;
        DLB_TRY(optimizer_step_sink(m->ctx, m->optimizer, &k, m->params + o, m->grads + o, m->m1 + o, m->m2 + o,
                                    m->m2hat ? m->m2hat + o : nullptr, wd != 0.f ? m->wd_mask + o : nullptr,
                                    (int)l.units, (int)l.fan_in, job.sink));
      } else {
        DLB_TRY(segment(l.first_conn, nw, reinterpret_cast<unsigned *>(job.sink.slot) + 2));
      }
      DLB_TRY(planes_close(m->ctx, job));
      at = l.first_conn + nw;
    }
    DLB_TRY(segment(at, m->total_parameters - at, nullptr));
  } else {
    DLB_TRY(segment(0, m->total_parameters, nullptr));
  }
  // Recurrent weights of every IndRNN layer back into the layer's bounds
  // (Update_Weight_Regularization__Constraint_Recurrent_Weight,
  // v1/ops/constraints/constraint.cpp L:245-289).
  for (LayerRT &l : m->layers) {
    if (!is_indrnn(l)) continue;
    float lo, hi;
    recurrent_bounds(m, l, &lo, &hi);
    if (lo != 0.f || hi != 0.f)
      DLB_TRY(dlb_indrnn_clamp(m->ctx, m->params + l.first_recurrent, (int)l.units, lo, hi));
  }
  m->grads_clean = true;  // the update kernel clears every gradient it consumes
  m->params_lo_valid = fused;
  return DLB_OK;
}

// ref: Model::set_clip_gradient (v1/ops/constraints/clip_gradient.cpp L:30-73).
dlb_status dlb_model_set_clip_gradient(dlb_model *m, int use, float value) {
  DLB_REQUIRE(m && value > 0.f, "set_clip_gradient: the norm must be positive");
  m->use_clip_gradient = use != 0;
  m->clip_gradient = value;
  return DLB_OK;
}

// ref: Model::Set__Regularization__Constraint_Recurrent_Weight(index, lower,
// upper) (v1/ops/constraints/constraint.cpp L:143-243): a hidden recurrent layer,
// lower <= upper; 0 / 0 takes the clamp off.  Bounds equal to the default (within
// 1e-8, the reference's own test, L:41-57) keep following clip_gradient.
dlb_status dlb_model_set_constraint_recurrent_weight(dlb_model *m, size_t layer, float lower, float upper) {
  DLB_REQUIRE(m && layer > 0 && layer + 1 < m->layers.size(),
              "set_constraint_recurrent_weight: the layer must be a hidden layer");
  LayerRT &l = m->layers[layer];
  if (!is_indrnn(l)) {
    set_error("set_constraint_recurrent_weight: layer %zu has no recurrent weights", layer);
    return DLB_ERR_INVALID;
  }
  DLB_REQUIRE(lower <= upper, "set_constraint_recurrent_weight: lower bound above upper bound");
  l.rec_custom = false;
  float dlo, dhi;
  recurrent_bounds(m, l, &dlo, &dhi);
  const bool is_default = fabsf(lower - dlo) <= 1e-8f && fabsf(upper - dhi) <= 1e-8f;
  l.rec_custom = !is_default;
  l.rec_lower = lower;
  l.rec_upper = upper;
  return DLB_OK;
}

// ref: Set__Regularization__Constraint_Recurrent_Weight__Default (L:97-141).
dlb_status dlb_model_set_constraint_recurrent_weight_default(dlb_model *m, size_t layer) {
  DLB_REQUIRE(m && layer > 0 && layer + 1 < m->layers.size(),
              "set_constraint_recurrent_weight_default: the layer must be a hidden layer");
  if (!is_indrnn(m->layers[layer])) {
    set_error("set_constraint_recurrent_weight_default: layer %zu has no recurrent weights", layer);
    return DLB_ERR_INVALID;
  }
  m->layers[layer].rec_custom = false;
  return DLB_OK;
}

dlb_status dlb_model_get_constraint_recurrent_weight(dlb_model *m, size_t layer, float *lower, float *upper) {
  DLB_REQUIRE(m && lower && upper && layer < m->layers.size(), "get_constraint_recurrent_weight");
  *lower = *upper = 0.f;
  if (is_indrnn(m->layers[layer])) recurrent_bounds(m, m->layers[layer], lower, upper);
  return DLB_OK;
}

dlb_status dlb_model_reset_loss(dlb_model *m) {
  DLB_REQUIRE(m, "null");
  m->loss_rows = 0;
  if (m->loss_sum) DLB_TRY(dlb_memset(m->ctx, m->loss_sum, 0, sizeof(double)));
  if (m->accu_sum) DLB_TRY(dlb_memset(m->ctx, m->accu_sum, 0, sizeof(double)));
  return DLB_OK;
}

// ref: Model::type_state_propagation as Driver::evalt / Driver::train set it
// (drivers/driver.cpp L:63, L:111).
dlb_status dlb_model_set_propagation(dlb_model *m, int state) {
  DLB_REQUIRE(m && (state == DLB_PROPAGATION_INFERENCE || state == DLB_PROPAGATION_TRAINING), "set_propagation");
  m->propagation = state;
  return DLB_OK;
}

// ref: Model::set_accu_fn (v1/learner/train.cpp L:63-75), Model::acc_var.
dlb_status dlb_model_set_accu_fn(dlb_model *m, int fn) {
  DLB_REQUIRE(m, "null");
  if (fn != DLB_ACCU_CROSS_ENTROPY && fn != DLB_ACCU_DISTANCE) {
    set_error("set_accu_fn: accuracy function %d is outside the supported set (CROSS_ENTROPY, DISTANCE)", fn);
    return DLB_ERR_UNSUPPORTED;
  }
  m->accu_fn = fn;
  return DLB_OK;
}
dlb_status dlb_model_set_accu_var(dlb_model *m, float v) {
  DLB_REQUIRE(m && v >= 0.f, "set_accu_var");
  m->accu_var = v;
  return DLB_OK;
}

// ref: Model::compute_loss (v1/learner/compute_loss.cpp L:140-161).
dlb_status dlb_model_compute_loss_device(dlb_model *m, size_t rows, const float *Y_dev) {
  DLB_REQUIRE(m && Y_dev && rows > 0 && rows <= m->alloc_rows, "compute_loss_device");
  LayerRT &o = m->layers.back();
  if (time_stepped(m)) {
    // Time steps t >= n_time_delay of every row (compute_loss_rec_mp,
    // v1/learner/compute_loss_mp.cpp L:115-205).
    DLB_REQUIRE(Y_dev != m->target, "compute_loss_device: target aliases the model's own buffer");
    const size_t T = m->seq_w, d = m->n_time_delay, W = o.units;
    DLB_TRY(dlb_time_major(m->ctx, Y_dev, m->target, nullptr, (int)rows, (int)T, (int)W));
    const size_t skip = d * rows * W;
    DLB_TRY(dlb_loss_eval(m->ctx, m->loss, m->accu_fn, m->accu_var, o.A + skip, m->target + skip,
                          (int)((T - d) * rows), (int)W, m->loss_sum, m->accu_sum));
    m->loss_rows += rows * (T - d);
    return DLB_OK;
  }
  DLB_TRY(dlb_loss_eval(m->ctx, m->loss, m->accu_fn, m->accu_var, o.A, Y_dev, (int)rows, (int)o.units,
                        m->loss_sum, m->accu_sum));
  m->loss_rows += rows;
  return DLB_OK;
}
dlb_status dlb_model_compute_loss(dlb_model *m, size_t rows, const float *const *Ym) {
  DLB_REQUIRE(m && Ym && rows > 0 && rows <= m->alloc_rows, "compute_loss");
  float *dst = time_stepped(m) ? m->target_rows : m->target;
  DLB_TRY(stage_rows(m, 1, &m->stage_y, &m->stage_y_elems, rows, m->seq_w * n_out(m), Ym, dst));
  DLB_TRY(dlb_model_compute_loss_device(m, rows, dst));
  return rows_consumed(m, 1);
}

// Percent of trials since reset_loss, over every rank's rows
// (Model::get_accu, v1/learner/metrics.cpp L:89-114; n_acc_trial as
// Driver::evalt sets it, drivers/driver.cpp L:95-99).
dlb_status dlb_model_get_accuracy(dlb_model *m, double *accuracy) {
  DLB_REQUIRE(m && accuracy && m->accu_sum, "get_accuracy");
  void *scr = nullptr;
  DLB_TRY(scratch(m->ctx, sizeof(double), &scr));
  double *tmp = static_cast<double *>(scr);
  DLB_TRY(dlb_memcpy_d2d(m->ctx, tmp, m->accu_sum, sizeof(double)));
  DLB_TRY(dlb_allreduce_f64(m->ctx, tmp, 1));
  double s = 0.0;
  DLB_TRY(dlb_memcpy_d2h(m->ctx, &s, tmp, sizeof(double)));
  const double trials = (double)m->loss_rows * (double)dlb_comm_world(m->ctx) *
                        (m->accu_fn == DLB_ACCU_CROSS_ENTROPY ? 1.0 : (double)n_out(m));
  *accuracy = trials == 0.0 ? 0.0 : s / trials * 100.0;
  return DLB_OK;
}

// MSE: sum / (rows * n_out); cross-entropy: sum / rows (v1/learner/loss.cpp
// L:158-221), over every rank's rows.
dlb_status dlb_model_get_loss(dlb_model *m, double *loss) {
  DLB_REQUIRE(m && loss && m->loss_sum, "get_loss");
  void *scr = nullptr;
  DLB_TRY(scratch(m->ctx, sizeof(double), &scr));
  double *tmp = static_cast<double *>(scr);
  DLB_TRY(dlb_memcpy_d2d(m->ctx, tmp, m->loss_sum, sizeof(double)));
  DLB_TRY(dlb_allreduce_f64(m->ctx, tmp, 1));
  double s = 0.0;
  DLB_TRY(dlb_memcpy_d2h(m->ctx, &s, tmp, sizeof(double)));
  const double rows = (double)m->loss_rows * (double)dlb_comm_world(m->ctx);
  if (rows == 0) { *loss = 1.0; return DLB_OK; }
  *loss = m->loss == DLB_LOSS_CROSS_ENTROPY ? s / rows : s / (rows * (double)n_out(m));
  return DLB_OK;
}

static dlb_status update_and_merge_overlapped(dlb_model *m, size_t rows);

// Starts the trip of the current loss sum to the host (slot = step parity) and
// returns without waiting.
static dlb_status loss_capture(dlb_model *m, int slot) {
  DLB_REQUIRE(m->loss_sum, "loss: no step has run");
  if (!m->loss_tmp) {
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(&m->loss_tmp), 4 * sizeof(double)));
    DLB_TRY(dlb_host_alloc(reinterpret_cast<void **>(&m->loss_host), 4 * sizeof(double)));
    for (cudaEvent_t &e : m->loss_ready) DLB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  // Per slot {loss sum, accuracy counter}; the counter only when the training
  // pass keeps it.
  double *dev = m->loss_tmp + 2 * slot, *host = m->loss_host + 2 * slot;
  const size_t n = m->training_accuracy ? 2 : 1;
  DLB_TRY(dlb_memcpy_d2d(m->ctx, dev, m->loss_sum, sizeof(double)));
  if (n == 2) DLB_TRY(dlb_memcpy_d2d(m->ctx, dev + 1, m->accu_sum, sizeof(double)));
  DLB_TRY(dlb_allreduce_f64(m->ctx, dev, n));
  DLB_CUDA(cudaMemcpyAsync(host, dev, n * sizeof(double), cudaMemcpyDeviceToHost, m->ctx->stream));
  DLB_CUDA(cudaEventRecord(m->loss_ready[slot], m->ctx->stream));
  m->loss_rows_at[slot] = m->loss_rows;
  m->loss_valid[slot] = true;
  return DLB_OK;
}

// Waits for a captured loss and normalises it as dlb_model_get_loss does; the
// accuracy of the same step (percent, as dlb_model_get_accuracy) goes to
// m->step_accuracy when the training pass keeps the counter.
static dlb_status loss_collect(dlb_model *m, int slot, double *loss) {
  if (!m->loss_valid[slot]) {
    *loss = nan("");  // a lagged read before the first step has finished
    return DLB_OK;
  }
  DLB_CUDA(cudaEventSynchronize(m->loss_ready[slot]));
  const double rows = (double)m->loss_rows_at[slot] * (double)dlb_comm_world(m->ctx);
  const double s = m->loss_host[2 * slot];
  if (m->training_accuracy) {
    const double trials = rows * (m->accu_fn == DLB_ACCU_CROSS_ENTROPY ? 1.0 : (double)n_out(m));
    m->step_accuracy = trials == 0.0 ? 0.0 : m->loss_host[2 * slot + 1] / trials * 100.0;
  }
  if (rows == 0) { *loss = 1.0; return DLB_OK; }
  *loss = m->loss == DLB_LOSS_CROSS_ENTROPY ? s / rows : s / (rows * (double)n_out(m));
  return DLB_OK;
}

// Plain stack of fully connected layers (no residual block, one time step).
static bool plain_stack(const dlb_model *m) {
  if (time_stepped(m)) return false;
  for (const LayerRT &l : m->layers)
    if (l.type != DLB_LAYER_FULLY_CONNECTED || l.group != 0) return false;
  return true;
}

// Backward pass and weight gradients of a plain stack in one sweep, for
// multi-GPU steps: a layer's weight gradient is formed as soon as its error is
// final and its all-reduce starts on the second stream, so that the exchange
// overlaps the rest of the backward pass instead of only the later weight-
// gradient products.  Same kernels on the same operands as
// dlb_model_backward_pass followed by dlb_model_update_derivatives: the
// results are identical.
//
// Where every weight matrix divides by rows among the ranks, the exchange is a
// reduce-scatter and the update moves in here as well: once the product that
// reads the layer's weights has been enqueued, the rank updates the rows it
// owns (gradient, weights and moments of that slice only: 1 / world of the
// optimizer's traffic), the updated rows are gathered on the second stream,
// and the matrix is split into its planes one layer later, when the gather
// has had two products' time.  Same bytes over NVLink as the all-reduce.
static dlb_status backward_and_derivatives_overlapped(dlb_model *m, size_t rows, size_t update_rows,
                                                      size_t training_size) {
  const int B = (int)rows;
  const int accumulate = m->grads_clean ? 0 : 1;
  const bool shard = sharded_update_possible(m);
  OwnerUpdate owners(m);
  if (shard) DLB_TRY(owners.begin(update_rows, training_size));
  else DLB_TRY(gather_moments(m));
  for (size_t i = m->layers.size() - 1; i >= 1; --i) {
    LayerRT &l = m->layers[i];
    const int H = (int)l.units;
    if (i + 1 != m->layers.size() && !l.error_final) {  // hidden layer: l.delta holds dA
      if (l.norm != DLB_NORM_NONE) {
        DLB_TRY(norm_backward(m, l, l.delta, l.delta_lo, l.Z, l.A, l.af, B));
      } else {
        DLB_TRY(dlb_activation_backward(m->ctx, l.delta, l.Z, l.A, nullptr, l.af, B, H, nullptr));
        DLB_TRY(dlb_split_planes_2d(m->ctx, l.delta, l.delta_lo, B, H));
      }
    }
    l.error_final = false;
    const float *X = i == 1 ? m->input : m->layers[i - 1].A;
    const float *X_lo = i == 1 ? m->input_lo : m->layers[i - 1].A_lo;
    float *dbias = l.norm == DLB_NORM_NONE ? m->grads + l.first_bias : nullptr;
    DLB_TRY(fc_weight_gradient_lines(m->ctx, l.delta, l.delta_lo, X, X_lo, m->grads + l.first_conn, dbias,
                                     B, (int)l.fan_in, H, accumulate, class_error(m, i)));
    if (shard) {
      DLB_TRY(owners.reduce(l));
    } else {
      DLB_TRY(dlb_allreduce_f32_overlapped(m->ctx, m->grads + l.first_conn, l.last_conn - l.first_conn));
    }
    if (i > 1) {
      LayerRT &below = m->layers[i - 1];
      if (below.norm == DLB_NORM_NONE) {
        DLB_TRY(dlb_fc_backward_input_derivative(m->ctx, l.delta, l.delta_lo, m->params + l.first_conn,
                                                 m->params_lo + l.first_conn, below.Z, below.A, below.af,
                                                 below.delta, below.delta_lo, B, (int)l.fan_in, H));
        below.error_final = true;
      } else {
        DLB_TRY(dlb_fc_backward_input(m->ctx, l.delta, l.delta_lo, m->params + l.first_conn,
                                      m->params_lo + l.first_conn, below.delta, B, (int)l.fan_in, H));
      }
    }
    if (shard) DLB_TRY(owners.update(l));  // nothing reads this layer's weights any more in this step
    if (i == 1) break;
  }
  m->grads_clean = false;
  // Bias, gamma and beta gradients follow the weight blocks.
  DLB_TRY(dlb_allreduce_f32_overlapped(m->ctx, m->grads + m->total_weights,
                                       m->total_parameters - m->total_weights));
  DLB_TRY(owners.finish());
  return dlb_comm_join(m->ctx);
}

// Backward, weight gradients and their exchange inside a training step.
static dlb_status backward_update_merge(dlb_model *m, size_t rows) {
  DLB_REQUIRE(rows > 0 && rows <= m->alloc_rows, "train_step: rows");
  if (dlb_comm_world(m->ctx) > 1 && plain_stack(m)) {
    const size_t g = m->global_rows ? m->global_rows : rows;
    return backward_and_derivatives_overlapped(m, rows, g, m->training_size ? m->training_size : g);
  }
  DLB_TRY(dlb_model_backward_pass(m, rows));
  return update_and_merge_overlapped(m, rows);
}

static dlb_status update_and_merge_overlapped(dlb_model *m, size_t rows) {
  m->overlap_grad_allreduce = dlb_comm_world(m->ctx) > 1;
  dlb_status st;
  if (m->overlap_grad_allreduce && sharded_update_possible(m)) {
    // Residual stacks: the backward pass is complete, so each matrix is
    // reduce-scattered, updated by its owners and gathered right behind its
    // weight-gradient product.
    OwnerUpdate owners(m);
    const size_t g = m->global_rows ? m->global_rows : rows;
    st = owners.begin(g, m->training_size ? m->training_size : g);
    if (st == DLB_OK) st = update_derivatives_flat(m, rows, &owners);
  } else {
    st = m->overlap_grad_allreduce ? gather_moments(m) : DLB_OK;
    if (st == DLB_OK) st = dlb_model_update_derivatives(m, rows);
  }
  if (st == DLB_OK) st = dlb_model_merge_derivatives(m);
  m->overlap_grad_allreduce = false;
  return st;
}

dlb_status dlb_model_train_step_device(dlb_model *m, size_t rows, const float *X_dev,
                                       const float *Y_dev) {
  DLB_TRY(dlb_model_reset_loss(m));
  DLB_TRY(dlb_model_forward_pass_device(m, rows, X_dev));
  DLB_TRY(dlb_model_compute_error_device(m, rows, Y_dev));
  DLB_TRY(backward_update_merge(m, rows));
  const size_t g = m->global_rows ? m->global_rows : rows;
  return dlb_model_update_weights(m, g, m->training_size ? m->training_size : g);
}

dlb_status dlb_model_train_step(dlb_model *m, size_t rows, const float *X_host,
                                const float *Y_host, double *loss) {
  DLB_REQUIRE(m && X_host && Y_host && rows > 0, "train_step");
  DLB_TRY(check_supported(m));
  DLB_TRY(ensure_batch(m, rows));
  float *x_dev = time_stepped(m) ? m->input_rows : m->input;
  float *y_dev = time_stepped(m) ? m->target_rows : m->target;
  DLB_TRY(stage_block(m, &m->stage_x, &m->stage_x_elems, rows * m->seq_w * n_in(m), X_host, x_dev));
  DLB_TRY(stage_block(m, &m->stage_y, &m->stage_y_elems, rows * m->seq_w * n_out(m), Y_host, y_dev));
  DLB_TRY(dlb_model_reset_loss(m));
  DLB_TRY(dlb_model_forward_pass_device(m, rows, x_dev));
  DLB_TRY(dlb_model_compute_error_device(m, rows, y_dev));
  DLB_TRY(backward_update_merge(m, rows));
  // The loss starts its way to the host, the update is enqueued, and only then
  // does the host wait for the loss: the update runs meanwhile.
  const int slot = (int)(m->loss_steps++ & 1);
  if (loss) DLB_TRY(loss_capture(m, slot));
  const size_t g = m->global_rows ? m->global_rows : rows;
  DLB_TRY(dlb_model_update_weights(m, g, m->training_size ? m->training_size : g));
  if (loss) DLB_TRY(loss_collect(m, slot, loss));
  return DLB_OK;
}

// Input side of the mini-batch loop, MiniBatch::train_mp
// (v1/data/dataset/minibatch.cpp L:286-323): the reference hands each batch
// to the model as host rows; here the next batch crosses PCIe while the
// current one trains.
dlb_status dlb_model_stage_batch(dlb_model *m, size_t rows, const float *X_host, const float *Y_host) {
  DLB_REQUIRE(m && X_host && Y_host && rows > 0, "stage_batch");
  DLB_TRY(check_supported(m));
  DLB_REQUIRE(m->ahead_head - m->ahead_tail < 2, "stage_batch: two batches are staged already");
  DLB_CUDA(cudaSetDevice(m->ctx->device));
  if (!m->copy_stream) DLB_CUDA(cudaStreamCreateWithFlags(&m->copy_stream, cudaStreamNonBlocking));
  dlb_model::Ahead &a = m->ahead[m->ahead_head % 2];
  if (!a.ready) {
    DLB_CUDA(cudaEventCreateWithFlags(&a.ready, cudaEventDisableTiming));
    DLB_CUDA(cudaEventCreateWithFlags(&a.consumed, cudaEventDisableTiming));
  }
  // The step that read this slot last must be past its reads.
  if (a.in_use) DLB_CUDA(cudaStreamWaitEvent(m->copy_stream, a.consumed, 0));
  const size_t nx = rows * m->seq_w * n_in(m), ny = rows * m->seq_w * n_out(m);
  auto fit = [&](float **buf, size_t *have, size_t need) -> dlb_status {
    if (need <= *have) return DLB_OK;
    if (*buf) {
      DLB_CUDA(cudaStreamSynchronize(m->copy_stream));
      DLB_CUDA(cudaStreamSynchronize(m->ctx->stream));
      DLB_TRY(dlb_free(m->ctx, *buf));
    }
    *buf = nullptr;
    *have = 0;
    DLB_TRY(dlb_malloc(m->ctx, reinterpret_cast<void **>(buf), need * sizeof(float)));
    *have = need;
    return DLB_OK;
  };
  DLB_TRY(fit(&a.x, &a.x_elems, nx));
  DLB_TRY(fit(&a.y, &a.y_elems, ny));
  DLB_CUDA(cudaMemcpyAsync(a.x, X_host, nx * sizeof(float), cudaMemcpyHostToDevice, m->copy_stream));
  DLB_CUDA(cudaMemcpyAsync(a.y, Y_host, ny * sizeof(float), cudaMemcpyHostToDevice, m->copy_stream));
  DLB_CUDA(cudaEventRecord(a.ready, m->copy_stream));
  a.rows = rows;
  ++m->ahead_head;
  return DLB_OK;
}

dlb_status dlb_model_train_step_staged(dlb_model *m, double *loss) {
  DLB_REQUIRE(m, "train_step_staged");
  DLB_REQUIRE(m->ahead_head > m->ahead_tail, "train_step_staged: no batch has been staged");
  dlb_model::Ahead &a = m->ahead[m->ahead_tail % 2];
  ++m->ahead_tail;
  const size_t rows = a.rows;
  DLB_CUDA(cudaStreamWaitEvent(m->ctx->stream, a.ready, 0));
  DLB_TRY(dlb_model_reset_loss(m));
  DLB_TRY(dlb_model_forward_pass_device(m, rows, a.x));
  DLB_TRY(dlb_model_compute_error_device(m, rows, a.y));
  DLB_CUDA(cudaEventRecord(a.consumed, m->ctx->stream));
  a.in_use = true;
  DLB_TRY(backward_update_merge(m, rows));
  // The loss starts its way to the host and the update is enqueued before the
  // host waits for anything.  With a loss lag of one step the wait is for the
  // loss of the step before, which has long arrived: the host then never waits
  // for the step it has just enqueued and runs one step ahead of the device.
  const int slot = (int)(m->loss_steps++ & 1);
  if (loss) DLB_TRY(loss_capture(m, slot));
  const size_t g = m->global_rows ? m->global_rows : rows;
  DLB_TRY(dlb_model_update_weights(m, g, m->training_size ? m->training_size : g));
  if (loss) DLB_TRY(loss_collect(m, m->loss_lag ? slot ^ 1 : slot, loss));
  return DLB_OK;
}

dlb_status dlb_model_set_training_accuracy(dlb_model *m, int on) {
  DLB_REQUIRE(m, "set_training_accuracy");
  m->training_accuracy = on != 0;
  return DLB_OK;
}

dlb_status dlb_model_set_sharded_update(dlb_model *m, int on) {
  DLB_REQUIRE(m, "set_sharded_update");
  m->sharded_update = on != 0;
  return DLB_OK;
}

dlb_status dlb_model_set_loss_lag(dlb_model *m, int steps) {
  DLB_REQUIRE(m && (steps == 0 || steps == 1), "set_loss_lag: 0 or 1");
  m->loss_lag = steps;
  return DLB_OK;
}

dlb_status dlb_model_get_layer_outputs(dlb_model *m, size_t layer, size_t rows, float *host_out) {
  DLB_REQUIRE(m && host_out && layer_at(m, layer) && rows <= m->alloc_rows, "get_layer_outputs");
  const LayerRT &l = m->layers[layer];
  const float *src = layer == 0 ? m->input : l.A;
  DLB_REQUIRE(src, "get_layer_outputs: no forward pass yet");
  const size_t w = layer == 0 ? n_in(m) : l.units;
  return dlb_memcpy_d2h(m->ctx, host_out, src, rows * w * m->seq_w * sizeof(float));
}

dlb_status dlb_model_get_layer_errors(dlb_model *m, size_t layer, size_t rows, int which,
                                      float *host_out) {
  DLB_REQUIRE(m && host_out && layer_at(m, layer) && layer > 0 && rows <= m->alloc_rows,
              "get_layer_errors");
  (void)which;
  const LayerRT &l = m->layers[layer];
  DLB_REQUIRE(l.delta, "get_layer_errors: no backward pass yet");
  return dlb_memcpy_d2h(m->ctx, host_out, l.delta, rows * l.units * m->seq_w * sizeof(float));
}

}  // extern "C"
