// The reference's on-disk format: Model::save_params (dimensions, layers, every
// weight as text) and Model::save_spec_params (hyperparameters), written so
// that the reference's Model::load reads a model trained here, and read so
// that a model saved by the reference continues here
// (v1/learner/save.cpp L:34-760, v1/learner/load.cpp).  Host code only; the
// flat vectors cross PCIe once through the library's own copy entry points.
//
// Numbers are printed as the reference prints them: a float widened to double
// through an output stream with 16 significant digits, lines ended by CR LF.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <fstream>
#include <iomanip>
#include <limits>
#include <sstream>
#include <string>
#include <vector>

#include "common.cuh"
#include "model.cuh"

using namespace dlb;

namespace {

const char *const CRLF = "\r\n";

std::string num(float v) {
  std::ostringstream s;
  s << std::setprecision(16) << v;
  return s.str();
}
std::string num(double v) {
  std::ostringstream s;
  s << std::setprecision(16) << v;
  return s.str();
}
std::string num(size_t v) { return std::to_string(v); }
std::string num(int v) { return std::to_string(v); }

bool fc_like(const LayerRT &l) {
  return l.type == DLB_LAYER_FULLY_CONNECTED || l.type == DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT;
}
bool indrnn(const LayerRT &l) { return l.type == DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT; }

// Model::Activation_Function__To__Class_Activation_Function (v1/learner/train.cpp
// L:313-362) over the supported activations; 0 where none has been set.
int activation_class(int af) {
  switch (af) {
    case DLB_AF_ELU: case DLB_AF_ISRLU: case DLB_AF_LINEAR: return 1;  // ASYMMETRIC
    case DLB_AF_LEAKY_RELU: case DLB_AF_RELU: return 2;                // RECTIFIER
    case DLB_AF_SELU: return 3;                                        // SELF_NORMALIZATION
    case DLB_AF_SOFTMAX: return 4;                                     // SOFTMAX
    default: return 0;
  }
}
// An activation of the class, for a layer that stores its class only (the first
// layer of a residual block has no activation units of its own).
int activation_of_class(int cls) {
  switch (cls) {
    case 1: return DLB_AF_LINEAR;
    case 2: return DLB_AF_RELU;
    case 3: return DLB_AF_SELU;
    case 4: return DLB_AF_SOFTMAX;
    default: return 0;
  }
}

// The layer whose outputs layer i reads (Layer::previous_connected_layers[0]):
// the layer before it in the list, or, for the first layer of a residual block,
// the layer before the block's RESIDUAL entry; a block that has ended is read
// through its RESIDUAL entry.
size_t source_layer(const dlb_model *m, size_t i) {
  size_t p = i - 1;
  if (m->layers[p].type == DLB_LAYER_RESIDUAL && m->layers[i].group == 1 && m->layers[i].block_input) --p;
  // p may now sit on the last layer of an earlier block: that block is read
  // through its RESIDUAL entry.
  if (m->layers[p].group == 1 && !(m->layers[i].group == 1 && !m->layers[i].block_input)) {
    size_t q = p;
    while (m->layers[q].type != DLB_LAYER_RESIDUAL) --q;
    p = q;
  }
  return p;
}

// First index of a layer's units in the reference's global arrays of neuron
// units (fully connected and IndRNN layers, the input layer included), basic
// units (RESIDUAL layers) and IndRNN activation units.
struct UnitBase {
  std::vector<size_t> neuron, basic, ind;
};
UnitBase unit_bases(const dlb_model *m) {
  UnitBase b;
  size_t n = 0, s = 0, r = 0;
  for (const LayerRT &l : m->layers) {
    b.neuron.push_back(n);
    b.basic.push_back(s);
    b.ind.push_back(r);
    if (fc_like(l)) n += l.units;
    if (l.type == DLB_LAYER_RESIDUAL) s += l.units;
    if (indrnn(l)) r += l.units;
  }
  return b;
}

void dropout_lines(std::string &out, const LayerRT &l, bool hidden) {
  out += "    type_dropout " + num(l.dropout) + CRLF;
  if (hidden) out += std::string("      use_coded_dropout 0") + CRLF;
  out += "      dropout_values[0] " + num(l.dropout_value) + CRLF;
  out += std::string("      dropout_values[1] 0") + CRLF;
  out += std::string("      dropout_values[2] 0") + CRLF;
}

struct HostState {
  std::vector<float> params;
  std::vector<std::vector<float>> mean_avg, sigma_avg;  // per layer, [T * units]
};

dlb_status fetch(dlb_model *m, HostState *h) {
  h->params.resize(m->total_parameters);
  DLB_TRY(dlb_model_get_array(m, "parameters", h->params.data(), m->total_parameters));
  h->mean_avg.resize(m->layers.size());
  h->sigma_avg.resize(m->layers.size());
  for (size_t i = 0; i < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    if (l.norm == DLB_NORM_NONE) continue;
    const size_t n = m->seq_w * l.norm_units;
    h->mean_avg[i].resize(n);
    h->sigma_avg[i].resize(n);
    DLB_TRY(dlb_model_get_layer_norm(m, i, "mean_average", h->mean_avg[i].data(), n));
    DLB_TRY(dlb_model_get_layer_norm(m, i, "variance_average", h->sigma_avg[i].data(), n));
  }
  return DLB_OK;
}

size_t gamma_at(const dlb_model *m, const LayerRT &l) { return m->total_weights + m->total_bias + l.first_norm_unit; }
size_t beta_at(const dlb_model *m, const LayerRT &l) { return gamma_at(m, l) + m->total_norm_units; }

// Information__Layer__Normalization (save.cpp L:523-590).
void normalization_lines(std::string &out, const dlb_model *m, size_t i, const HostState &h) {
  const LayerRT &l = m->layers[i];
  out += "    type_normalization " + num(l.norm) + CRLF;
  if (l.type != DLB_LAYER_RESIDUAL) out += std::string("      use_layer_normalization_before_activation 1") + CRLF;
  // Normalized units exist for every layer as soon as one layer is normalised,
  // and for none otherwise: as many as the layer has units, a block layer as
  // many as it has inputs (it normalises its input), a RESIDUAL layer as many
  // as its block puts out.
  const size_t n = m->any_norm ? l.norm_units : 0;
  out += "      number_normalized_units " + num(n) + CRLF;
  for (size_t k = 0; k < n; ++k) {
    out += "        NormU[" + num(k) + "]" + CRLF;
    if (l.norm == DLB_NORM_NONE) continue;
    out += "          scale " + num(h.params[gamma_at(m, l) + k]) + CRLF;
    out += "          shift " + num(h.params[beta_at(m, l) + k]) + CRLF;
    for (size_t t = 0; t < m->seq_w; ++t) {
      out += "          mean_average[" + num(t) + "] " + num(h.mean_avg[i][n * t + k]) + CRLF;
      out += "          variance_average[" + num(t) + "] " + num(h.sigma_avg[i][n * t + k]) + CRLF;
    }
  }
}

// Information__Layer__FC / Information__Output_Layer (save.cpp L:592-671).
void neuron_lines(std::string &out, const dlb_model *m, size_t i, const HostState &h, const UnitBase &base) {
  const LayerRT &l = m->layers[i];
  const size_t src = source_layer(m, i);
  const bool from_basic = m->layers[src].type == DLB_LAYER_RESIDUAL;
  const char *label = from_basic ? "connected_to_basic " : "connected_to_neuron ";
  const size_t first = from_basic ? base.basic[src] : base.neuron[src];
  for (size_t k = 0; k < l.units; ++k) {
    out += "      Neuron_unit[" + num(k) + "]" + CRLF;
    out += "        number_connections " + num(l.fan_in) + CRLF;
    for (size_t c = 0; c < l.fan_in; ++c) {
      const size_t w = l.first_conn + k * l.fan_in + c;
      out += std::string("          ") + label + num(first + c) + CRLF;
      out += "          weight[" + num(w) + "] " + num(h.params[w]) + CRLF;
    }
  }
}

void af_lines(std::string &out, const LayerRT &l) {
  const size_t n = (l.group == 1 && l.block_input) ? 0 : l.units;
  out += "    number_AF_units " + num(n) + CRLF;
  for (size_t k = 0; k < n; ++k) {
    out += "      AF[" + num(k) + "]" + CRLF;
    out += "        activation_function " + num(l.af) + CRLF;
  }
}

void bias_lines(std::string &out, const LayerRT &l, const HostState &h) {
  const size_t n = l.last_bias - l.first_bias;
  out += "    number_bias_parameters " + num(n) + CRLF;
  for (size_t k = 0; k < n; ++k) out += "      weight[" + num(l.first_bias + k) + "] " + num(h.params[l.first_bias + k]) + CRLF;
}

dlb_status write_file(const char *path, const std::string &text) {
  FILE *f = fopen(path, "wb");
  if (!f) {
    set_error("checkpoint: cannot open %s for writing", path);
    return DLB_ERR_INVALID;
  }
  const bool ok = fwrite(text.data(), 1, text.size(), f) == text.size();
  if (fclose(f) != 0 || !ok) {
    set_error("checkpoint: write to %s failed", path);
    return DLB_ERR_INVALID;
  }
  return DLB_OK;
}

// ---- reading -------------------------------------------------------------------

struct Reader {
  std::vector<std::string> lines;
  size_t at = 0;
  std::string path;

  dlb_status open(const char *p) {
    path = p;
    std::ifstream f(p, std::ios::in | std::ios::binary);
    if (!f.is_open()) {
      set_error("checkpoint: cannot open %s", p);
      return DLB_ERR_INVALID;
    }
    std::string line;
    while (std::getline(f, line)) {
      while (!line.empty() && (line.back() == '\r' || line.back() == ' ')) line.pop_back();
      size_t b = 0;
      while (b < line.size() && line[b] == ' ') ++b;
      if (b < line.size()) lines.push_back(line.substr(b));
    }
    return DLB_OK;
  }
  dlb_status fail(const std::string &want) {
    set_error("checkpoint: %s line %zu: expected `%s`, found `%s`", path.c_str(), at + 1, want.c_str(),
              at < lines.size() ? lines[at].c_str() : "<end of file>");
    return DLB_ERR_INVALID;
  }
  // A line that is exactly `text`.
  dlb_status expect(const std::string &text) {
    if (at >= lines.size() || lines[at] != text) return fail(text);
    ++at;
    return DLB_OK;
  }
  // A line `key value`.
  dlb_status value(const std::string &key, std::string *out) {
    if (at >= lines.size() || lines[at].compare(0, key.size() + 1, key + " ") != 0) return fail(key + " <value>");
    *out = lines[at].substr(key.size() + 1);
    ++at;
    return DLB_OK;
  }
  dlb_status real(const std::string &key, double *out) {
    std::string v;
    DLB_TRY(value(key, &v));
    if (v == "inf") *out = std::numeric_limits<double>::infinity();
    else if (v == "-inf") *out = -std::numeric_limits<double>::infinity();
    else *out = strtod(v.c_str(), nullptr);
    return DLB_OK;
  }
  dlb_status count(const std::string &key, size_t *out) {
    std::string v;
    DLB_TRY(value(key, &v));
    *out = (size_t)strtoull(v.c_str(), nullptr, 10);
    return DLB_OK;
  }
  bool peek(const std::string &prefix) const {
    return at < lines.size() && lines[at].compare(0, prefix.size(), prefix) == 0;
  }
};

struct LoadedLayer {
  int type = 0, cls = 0, af = 0, norm = 0, dropout = 0;
  double dropout_value = 0;
  double rec_lower = 0, rec_upper = 0;  // bounds of the recurrent weights
  size_t units = 0, depth = 0;
  std::vector<float> scale, shift, mean_avg, sigma_avg;  // norm: [units], [units], [T*units] x 2
  std::vector<std::pair<size_t, float>> weights;         // (index in the flat vector, value)
};

dlb_status read_dropout(Reader &r, LoadedLayer *l, bool hidden) {
  size_t v;
  DLB_TRY(r.count("type_dropout", &v));
  l->dropout = (int)v;
  if (hidden) DLB_TRY(r.count("use_coded_dropout", &v));
  double d;
  DLB_TRY(r.real("dropout_values[0]", &l->dropout_value));
  DLB_TRY(r.real("dropout_values[1]", &d));
  DLB_TRY(r.real("dropout_values[2]", &d));
  return DLB_OK;
}

dlb_status read_normalization(Reader &r, LoadedLayer *l, size_t T, bool residual) {
  size_t v, n;
  DLB_TRY(r.count("type_normalization", &v));
  l->norm = (int)v;
  if (!residual) DLB_TRY(r.count("use_layer_normalization_before_activation", &v));
  DLB_TRY(r.count("number_normalized_units", &n));
  if (l->norm != DLB_NORM_NONE) {
    l->scale.resize(n);
    l->shift.resize(n);
    l->mean_avg.resize(n * T);
    l->sigma_avg.resize(n * T);
  }
  for (size_t k = 0; k < n; ++k) {
    DLB_TRY(r.expect("NormU[" + num(k) + "]"));
    if (l->norm == DLB_NORM_NONE) continue;
    double d;
    DLB_TRY(r.real("scale", &d));
    l->scale[k] = (float)d;
    DLB_TRY(r.real("shift", &d));
    l->shift[k] = (float)d;
    for (size_t t = 0; t < T; ++t) {
      DLB_TRY(r.real("mean_average[" + num(t) + "]", &d));
      l->mean_avg[n * t + k] = (float)d;
      DLB_TRY(r.real("variance_average[" + num(t) + "]", &d));
      l->sigma_avg[n * t + k] = (float)d;
    }
  }
  return DLB_OK;
}

dlb_status read_weight(Reader &r, LoadedLayer *l) {
  if (!r.peek("weight[")) return r.fail("weight[<index>] <value>");
  const std::string &line = r.lines[r.at];
  const size_t close = line.find(']');
  if (close == std::string::npos || close + 2 > line.size()) return r.fail("weight[<index>] <value>");
  const size_t index = (size_t)strtoull(line.c_str() + 7, nullptr, 10);
  l->weights.emplace_back(index, (float)strtod(line.c_str() + close + 2, nullptr));
  ++r.at;
  return DLB_OK;
}

dlb_status read_neurons(Reader &r, LoadedLayer *l) {
  for (size_t k = 0; k < l->units; ++k) {
    DLB_TRY(r.expect("Neuron_unit[" + num(k) + "]"));
    size_t c;
    DLB_TRY(r.count("number_connections", &c));
    for (size_t j = 0; j < c; ++j) {
      if (!r.peek("connected_to_")) return r.fail("connected_to_<kind> <index>");
      ++r.at;
      DLB_TRY(read_weight(r, l));
    }
  }
  return DLB_OK;
}

dlb_status read_afs(Reader &r, LoadedLayer *l) {
  size_t n, v;
  DLB_TRY(r.count("number_AF_units", &n));
  for (size_t k = 0; k < n; ++k) {
    DLB_TRY(r.expect("AF[" + num(k) + "]"));
    DLB_TRY(r.count("activation_function", &v));
    if (k == 0) l->af = (int)v;
  }
  if (n == 0) l->af = activation_of_class(l->cls);
  return DLB_OK;
}

dlb_status read_bias(Reader &r, LoadedLayer *l) {
  size_t n;
  DLB_TRY(r.count("number_bias_parameters", &n));
  for (size_t k = 0; k < n; ++k) DLB_TRY(read_weight(r, l));
  return DLB_OK;
}

}  // namespace

extern "C" {

dlb_status dlb_model_save_params(dlb_model *m, const char *path) {
  DLB_REQUIRE(m && path && m->layers.size() >= 2, "save_params");
  for (const LayerRT &l : m->layers)
    if (l.type == DLB_LAYER_LSTM) {
      set_error("save_params: writing LSTM layers in the reference's format is not supported");
      return DLB_ERR_UNSUPPORTED;
    }
  HostState h;
  DLB_TRY(fetch(m, &h));
  const UnitBase base = unit_bases(m);
  size_t neurons = 0, basics = 0, afs = 0, inds = 0, all_units = 0;
  for (const LayerRT &l : m->layers) {
    all_units += l.norm_units;
    if (fc_like(l)) neurons += l.units;
    if (l.type == DLB_LAYER_RESIDUAL) basics += l.units;
    if (indrnn(l)) inds += l.units;
    else if (fc_like(l) && !(l.group == 1 && l.block_input)) afs += l.units;
  }
  std::string out;
  out.reserve(64 * m->total_parameters + 4096);
  out += std::string("|===| DIMENSION |===|") + CRLF;
  out += "type " + num(m->model_type) + CRLF;
  out += "number_layers " + num(m->layers.size()) + CRLF;
  out += "seq_w " + num(m->seq_w) + CRLF;
  out += "n_time_delay " + num(m->n_time_delay) + CRLF;
  out += std::string("use_first_layer_as_input 1") + CRLF;
  out += std::string("use_last_layer_as_output 1") + CRLF;
  out += "total_basic_units " + num(basics) + CRLF;
  out += std::string("total_basic_indice_units 0") + CRLF;
  out += "total_neuron_units " + num(neurons) + CRLF;
  out += "total_AF_units " + num(afs) + CRLF;
  out += "total_AF_Ind_recurrent_units " + num(inds) + CRLF;
  out += std::string("total_block_units 0") + CRLF;
  out += std::string("total_cell_units 0") + CRLF;
  out += "total_normalized_units " + num(m->any_norm ? all_units : 0) + CRLF;
  out += "total_parameters " + num(m->total_parameters) + CRLF;
  out += "total_weights " + num(m->total_weights) + CRLF;
  out += "total_bias " + num(m->total_bias) + CRLF;

  const LayerRT &in = m->layers.front();
  out += std::string("  Input layer:") + CRLF;
  out += "    type_layer " + num(in.type) + CRLF;
  out += "    type_activation " + num(activation_class(in.af)) + CRLF;
  dropout_lines(out, in, false);
  out += "    n_inp " + num(in.units) + CRLF;

  const float bound = powf(fminf(fmaxf(m->clip_gradient, 2.f), 10.f), 1.f / (float)m->seq_w);
  for (size_t i = 1; i + 1 < m->layers.size(); ++i) {
    const LayerRT &l = m->layers[i];
    out += "  Hidden layer " + num(i) + ":" + CRLF;
    out += "    type_layer " + num(l.type) + CRLF;
    out += std::string("    use_bidirectional 0") + CRLF;
    if (l.type == DLB_LAYER_RESIDUAL) {
      out += "    block_depth " + num(l.depth) + CRLF;
      out += "    padding " + num(l.pad) + CRLF;
      dropout_lines(out, l, true);
      normalization_lines(out, m, i, h);
      out += "    number_basic_units " + num(l.units) + CRLF;
      continue;
    }
    out += "    type_activation " + num(activation_class(l.af)) + CRLF;
    dropout_lines(out, l, true);
    normalization_lines(out, m, i, h);
    out += std::string("    use_tied_parameter 0") + CRLF;
    out += std::string("    k_sparsity 0") + CRLF;
    out += std::string("    alpha_sparsity 1") + CRLF;
    out += "    constraint_recurrent_weight_lower_bound " + num(indrnn(l) ? (l.rec_custom ? l.rec_lower : -bound) : 0.f) + CRLF;
    out += "    constraint_recurrent_weight_upper_bound " + num(indrnn(l) ? (l.rec_custom ? l.rec_upper : bound) : 0.f) + CRLF;
    out += "    number_neuron_units " + num(l.units) + CRLF;
    neuron_lines(out, m, i, h, base);
    if (indrnn(l)) {
      out += "    number_AF_Ind_recurrent_units " + num(l.units) + CRLF;
      for (size_t k = 0; k < l.units; ++k) {
        out += "      AF_Ind_R[" + num(k) + "]" + CRLF;
        out += "        activation_function " + num(l.af) + CRLF;
        out += "        connected_to_AF_Ind_R " + num(base.ind[i] + k) + CRLF;
        out += "        weight[" + num(l.first_recurrent + k) + "] " + num(h.params[l.first_recurrent + k]) + CRLF;
      }
    } else {
      af_lines(out, l);
    }
    bias_lines(out, l, h);
  }

  const size_t last = m->layers.size() - 1;
  const LayerRT &o = m->layers[last];
  out += std::string("  Output layer:") + CRLF;
  out += "    type_layer " + num(o.type) + CRLF;
  out += "    type_activation " + num(activation_class(o.af)) + CRLF;
  out += "    n_out " + num(o.units) + CRLF;
  neuron_lines(out, m, last, h, base);
  af_lines(out, o);
  bias_lines(out, o, h);
  out += std::string("|END| DIMENSION |END|") + CRLF;
  return write_file(path, out);
}

dlb_status dlb_model_save_spec_params(dlb_model *m, const char *path) {
  DLB_REQUIRE(m && path, "save_spec_params");
  const HParams &p = m->hp;
  const double inf = std::numeric_limits<double>::infinity();
  std::string out;
  auto section = [&](const char *name) { out += std::string("|===| ") + name + " |===|" + CRLF; };
  auto end = [&](const char *name, bool blank = true) {
    out += std::string("|END| ") + name + " |END|" + CRLF;
    if (blank) out += CRLF;
  };
  auto kv = [&](const char *key, const std::string &v) { out += std::string(key) + " " + v + CRLF; };
  // Values of optimizers and options outside the supported path are written as
  // the reference's defaults (model.hpp L:3020-3060), so that its loader finds
  // every key.
  section("GRADIENT DESCENT PARAMETERS");
  kv("learning_rate", num(p.learning_rate));
  kv("learning_rate_final", num(p.learning_rate_final));
  kv("learning_momentum", num(p.learning_momentum));
  kv("learning_gamma", num(p.learning_gamma));
  kv("use_nesterov", num((int)p.use_nesterov));
  end("GRADIENT DESCENT PARAMETERS");
  section("QUICKPROP PARAMETERS");
  kv("quickprop_decay", num(-0.0001f));
  kv("quickprop_mu", num(1.75f));
  end("QUICKPROP PARAMETERS");
  section("RESILLENT PROPAGATION PARAMETERS");
  kv("rprop_increase_factor", num(1.2f));
  kv("rprop_decrease_factor", num(0.5f));
  kv("rprop_delta_min", num(1e-6f));
  kv("rprop_delta_max", num(50.f));
  kv("rprop_delta_zero", num(0.1f));
  end("RESILLENT PROPAGATION PARAMETERS");
  section("SARPROP PARAMETERS");
  kv("sarprop_weight_decay_shift", num(-6.644f));
  kv("sarprop_step_error_threshold_factor", num(0.1f));
  kv("sarprop_step_error_shift", num(1.385f));
  kv("sarprop_temperature", num(0.015f));
  kv("sarprop_epoch", "0");
  end("SARPROP PARAMETERS");
  section("ADAM PARAMETERS");
  kv("adam_learning_rate", num(p.adam_learning_rate));
  kv("adam_beta1", num(p.adam_beta1));
  kv("adam_beta2", num(p.adam_beta2));
  kv("adam_epsilon", num(p.adam_epsilon));
  kv("adam_bias_correction", num((int)p.use_adam_bias_correction));
  kv("adam_gamma", num(p.adam_gamma));
  end("ADAM PARAMETERS");
  section("WARM RESTARTS PARAMETERS");
  kv("use_warm_restarts", "0");
  kv("warm_restarts_decay_learning_rate", "1");
  kv("warm_restarts_maximum_learning_rate", "1");
  kv("warm_restarts_minimum_learning_rate", num(1e-7f));
  kv("warm_restarts_initial_T_i", "1");
  kv("warm_restarts_multiplier", "2");
  end("WARM RESTARTS PARAMETERS");
  section("TRAINING PARAMETERS");
  kv("type_optimizer_function", num(m->optimizer));
  kv("type_loss_function", num(m->loss));
  kv("type_accuracy_function", num(m->accu_fn));
  kv("bit_fail_limit", "0.35");
  kv("pre_training_level", "0");
  kv("use_clip_gradient", num((int)m->use_clip_gradient));
  kv("clip_gradient", num(m->clip_gradient));
  end("TRAINING PARAMETERS");
  section("REGULARIZATION PARAMETERS");
  kv("regularization__max_norm_constraints", "0");
  kv("regularization__l1", "0");
  kv("regularization__l2", num(m->hp.regularization_l2));
  kv("regularization__srip", "0");
  kv("weight_decay", num(p.weight_decay));
  kv("use_normalized_weight_decay", num((int)p.use_normalized_weight_decay));
  end("REGULARIZATION PARAMETERS");
  section("NORMALIZATION PARAMETERS");
  kv("normalization_momentum_average", num(p.normalization_momentum_average));
  kv("normalization_epsilon", num(p.normalization_epsilon));
  kv("batch_renormalization_r_correction_maximum", num(p.brn_r_max));
  kv("batch_renormalization_d_correction_maximum", num(p.brn_d_max));
  end("NORMALIZATION PARAMETERS");
  section("LOSS PARAMETERS");
  kv("loss_train", num(inf));
  kv("loss_valid", num(inf));
  kv("loss_testg", num(inf));
  end("LOSS PARAMETERS");
  section("ACCURANCY PARAMETERS");
  kv("acc_var", num(m->accu_var));
  kv("acc_train", "0");
  kv("acc_valid", "0");
  kv("acc_testg", "0");
  end("ACCURANCY PARAMETERS");
  section("COMPUTATION PARAMETERS");
  kv("use_cu", "0");
  kv("use_mp", "1");
  kv("pct_threads", "100");
  kv("maximum_batch_size", num(m->max_batch));
  end("COMPUTATION PARAMETERS", false);
  return write_file(path, out);
}

// Model::load (v1/learner/load.cpp L:1243-): the dimension file builds the
// layers, the spec file sets the hyperparameters; `m` must be a fresh model.
dlb_status dlb_model_load(dlb_model *m, const char *path_params, const char *path_spec) {
  DLB_REQUIRE(m && path_params && path_spec, "load");
  DLB_REQUIRE(m->layers.empty(), "load: the model has been compiled already");
  Reader r;
  DLB_TRY(r.open(path_params));
  size_t type, n_layers, T, delay, v, total_parameters;
  DLB_TRY(r.expect("|===| DIMENSION |===|"));
  DLB_TRY(r.count("type", &type));
  DLB_TRY(r.count("number_layers", &n_layers));
  DLB_TRY(r.count("seq_w", &T));
  DLB_TRY(r.count("n_time_delay", &delay));
  for (const char *key : {"use_first_layer_as_input", "use_last_layer_as_output", "total_basic_units",
                          "total_basic_indice_units", "total_neuron_units", "total_AF_units",
                          "total_AF_Ind_recurrent_units", "total_block_units", "total_cell_units",
                          "total_normalized_units"})
    DLB_TRY(r.count(key, &v));
  DLB_TRY(r.count("total_parameters", &total_parameters));
  DLB_TRY(r.count("total_weights", &v));
  DLB_TRY(r.count("total_bias", &v));
  DLB_REQUIRE(n_layers >= 2 && T >= 1, "load: dimensions");

  std::vector<LoadedLayer> L(n_layers);
  DLB_TRY(r.expect("Input layer:"));
  DLB_TRY(r.count("type_layer", &v));
  L[0].type = (int)v;
  DLB_TRY(r.count("type_activation", &v));
  DLB_TRY(read_dropout(r, &L[0], false));
  DLB_TRY(r.count("n_inp", &L[0].units));
  for (size_t i = 1; i + 1 < n_layers; ++i) {
    LoadedLayer &l = L[i];
    DLB_TRY(r.expect("Hidden layer " + num(i) + ":"));
    DLB_TRY(r.count("type_layer", &v));
    l.type = (int)v;
    DLB_TRY(r.count("use_bidirectional", &v));
    if (l.type == DLB_LAYER_RESIDUAL) {
      DLB_TRY(r.count("block_depth", &l.depth));
      DLB_TRY(r.count("padding", &v));
      DLB_TRY(read_dropout(r, &l, true));
      DLB_TRY(read_normalization(r, &l, T, true));
      DLB_TRY(r.count("number_basic_units", &l.units));
      continue;
    }
    if (l.type != DLB_LAYER_FULLY_CONNECTED && l.type != DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT) {
      set_error("load: layer %zu has type %d, outside the supported path", i, l.type);
      return DLB_ERR_UNSUPPORTED;
    }
    DLB_TRY(r.count("type_activation", &v));
    l.cls = (int)v;
    DLB_TRY(read_dropout(r, &l, true));
    DLB_TRY(read_normalization(r, &l, T, false));
    double d;
    DLB_TRY(r.count("use_tied_parameter", &v));
    DLB_TRY(r.count("k_sparsity", &v));
    DLB_TRY(r.real("alpha_sparsity", &d));
    DLB_TRY(r.real("constraint_recurrent_weight_lower_bound", &l.rec_lower));
    DLB_TRY(r.real("constraint_recurrent_weight_upper_bound", &l.rec_upper));
    DLB_TRY(r.count("number_neuron_units", &l.units));
    DLB_TRY(read_neurons(r, &l));
    if (l.type == DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT) {
      size_t n;
      DLB_TRY(r.count("number_AF_Ind_recurrent_units", &n));
      for (size_t k = 0; k < n; ++k) {
        DLB_TRY(r.expect("AF_Ind_R[" + num(k) + "]"));
        DLB_TRY(r.count("activation_function", &v));
        l.af = (int)v;
        DLB_TRY(r.count("connected_to_AF_Ind_R", &v));
        DLB_TRY(read_weight(r, &l));
      }
    } else {
      DLB_TRY(read_afs(r, &l));
    }
    DLB_TRY(read_bias(r, &l));
  }
  LoadedLayer &o = L[n_layers - 1];
  DLB_TRY(r.expect("Output layer:"));
  DLB_TRY(r.count("type_layer", &v));
  o.type = (int)v;
  DLB_TRY(r.count("type_activation", &v));
  o.cls = (int)v;
  DLB_TRY(r.count("n_out", &o.units));
  DLB_TRY(read_neurons(r, &o));
  DLB_TRY(read_afs(r, &o));
  DLB_TRY(read_bias(r, &o));
  DLB_TRY(r.expect("|END| DIMENSION |END|"));

  // Build the model through its own construction entry points.
  std::vector<int> types(n_layers);
  std::vector<size_t> units(n_layers);
  for (size_t i = 0; i < n_layers; ++i) {
    types[i] = L[i].type;
    units[i] = L[i].type == DLB_LAYER_RESIDUAL ? L[i].depth : L[i].units;
  }
  DLB_TRY(dlb_model_compile(m, n_layers, T, (int)type, types.data(), units.data()));
  for (size_t i = 1; i < n_layers; ++i) {
    if (L[i].type == DLB_LAYER_RESIDUAL) continue;
    if (L[i].af != 0) DLB_TRY(dlb_model_set_layer_activation_function(m, i, L[i].af));
  }
  for (size_t i = 1; i + 1 < n_layers; ++i)
    if (L[i].norm != DLB_NORM_NONE) DLB_TRY(dlb_model_set_layer_normalization(m, i, L[i].norm));
  for (size_t i = 0; i + 1 < n_layers; ++i)
    if (L[i].dropout != DLB_DROPOUT_NONE)
      DLB_TRY(dlb_model_set_dropout(m, i, L[i].dropout, (float)L[i].dropout_value, 0));
  if (delay) DLB_TRY(dlb_model_set_seq_w(m, delay));

  // Hyperparameters.
  Reader s;
  DLB_TRY(s.open(path_spec));
  double d;
  auto skip_section = [&](const char *name, std::initializer_list<const char *> keys) -> dlb_status {
    DLB_TRY(s.expect(std::string("|===| ") + name + " |===|"));
    for (const char *k : keys) {
      std::string ignored;
      DLB_TRY(s.value(k, &ignored));
    }
    return s.expect(std::string("|END| ") + name + " |END|");
  };
  auto hparam = [&](const char *key, const char *name) -> dlb_status {
    DLB_TRY(s.real(key, &d));
    return dlb_model_set_hparam(m, name, d);
  };
  DLB_TRY(s.expect("|===| GRADIENT DESCENT PARAMETERS |===|"));
  DLB_TRY(hparam("learning_rate", "learning_rate"));
  DLB_TRY(hparam("learning_rate_final", "learning_rate_final"));
  DLB_TRY(hparam("learning_momentum", "learning_momentum"));
  DLB_TRY(hparam("learning_gamma", "learning_gamma"));
  DLB_TRY(hparam("use_nesterov", "use_nesterov"));
  DLB_TRY(s.expect("|END| GRADIENT DESCENT PARAMETERS |END|"));
  DLB_TRY(skip_section("QUICKPROP PARAMETERS", {"quickprop_decay", "quickprop_mu"}));
  DLB_TRY(skip_section("RESILLENT PROPAGATION PARAMETERS",
                       {"rprop_increase_factor", "rprop_decrease_factor", "rprop_delta_min", "rprop_delta_max",
                        "rprop_delta_zero"}));
  DLB_TRY(skip_section("SARPROP PARAMETERS",
                       {"sarprop_weight_decay_shift", "sarprop_step_error_threshold_factor",
                        "sarprop_step_error_shift", "sarprop_temperature", "sarprop_epoch"}));
  DLB_TRY(s.expect("|===| ADAM PARAMETERS |===|"));
  DLB_TRY(hparam("adam_learning_rate", "adam_learning_rate"));
  DLB_TRY(hparam("adam_beta1", "adam_beta1"));
  DLB_TRY(hparam("adam_beta2", "adam_beta2"));
  DLB_TRY(hparam("adam_epsilon", "adam_epsilon"));
  DLB_TRY(hparam("adam_bias_correction", "use_adam_bias_correction"));
  DLB_TRY(hparam("adam_gamma", "adam_gamma"));
  DLB_TRY(s.expect("|END| ADAM PARAMETERS |END|"));
  DLB_TRY(s.expect("|===| WARM RESTARTS PARAMETERS |===|"));
  DLB_TRY(s.real("use_warm_restarts", &d));
  if (d != 0.0) {
    set_error("load: warm restarts are outside the supported path");
    return DLB_ERR_UNSUPPORTED;
  }
  for (const char *k : {"warm_restarts_decay_learning_rate", "warm_restarts_maximum_learning_rate",
                        "warm_restarts_minimum_learning_rate", "warm_restarts_initial_T_i",
                        "warm_restarts_multiplier"})
    DLB_TRY(s.real(k, &d));
  DLB_TRY(s.expect("|END| WARM RESTARTS PARAMETERS |END|"));
  DLB_TRY(s.expect("|===| TRAINING PARAMETERS |===|"));
  DLB_TRY(s.real("type_optimizer_function", &d));
  DLB_TRY(dlb_model_set_optimizer(m, (int)d));
  DLB_TRY(s.real("type_loss_function", &d));
  DLB_TRY(dlb_model_set_loss_fn(m, (int)d));
  DLB_TRY(s.real("type_accuracy_function", &d));
  DLB_TRY(dlb_model_set_accu_fn(m, (int)d));
  DLB_TRY(s.real("bit_fail_limit", &d));
  DLB_TRY(s.real("pre_training_level", &d));
  double use_clip, clip;
  DLB_TRY(s.real("use_clip_gradient", &use_clip));
  DLB_TRY(s.real("clip_gradient", &clip));
  DLB_TRY(dlb_model_set_clip_gradient(m, use_clip != 0.0, (float)clip));
  // Bounds of the recurrent weights, now that the norm their default derives
  // from is known: the file's values, which stay the default when they equal it.
  for (size_t i = 1; i + 1 < n_layers; ++i)
    if (L[i].type == DLB_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT)
      DLB_TRY(dlb_model_set_constraint_recurrent_weight(m, i, (float)L[i].rec_lower, (float)L[i].rec_upper));
  DLB_TRY(s.expect("|END| TRAINING PARAMETERS |END|"));
  DLB_TRY(s.expect("|===| REGULARIZATION PARAMETERS |===|"));
  for (const char *k : {"regularization__max_norm_constraints", "regularization__l1", "regularization__l2",
                        "regularization__srip"}) {
    DLB_TRY(s.real(k, &d));
    if (std::string(k) == "regularization__l2") {
      DLB_TRY(dlb_model_set_l2(m, (float)d));
      continue;
    }
    if (d != 0.0) {
      set_error("load: %s = %g is outside the supported path", k, d);
      return DLB_ERR_UNSUPPORTED;
    }
  }
  DLB_TRY(s.real("weight_decay", &d));
  DLB_TRY(dlb_model_set_weight_decay(m, (float)d));
  DLB_TRY(hparam("use_normalized_weight_decay", "use_normalized_weight_decay"));
  DLB_TRY(s.expect("|END| REGULARIZATION PARAMETERS |END|"));
  DLB_TRY(s.expect("|===| NORMALIZATION PARAMETERS |===|"));
  DLB_TRY(s.real("normalization_momentum_average", &d));
  DLB_TRY(dlb_model_set_normalization_momentum_average(m, (float)d));
  DLB_TRY(s.real("normalization_epsilon", &d));
  DLB_TRY(dlb_model_set_normalization_epsilon(m, (float)d));
  DLB_TRY(s.real("batch_renormalization_r_correction_maximum", &d));
  DLB_TRY(dlb_model_set_brn_r_correction_maximum(m, (float)d));
  DLB_TRY(s.real("batch_renormalization_d_correction_maximum", &d));
  DLB_TRY(dlb_model_set_brn_d_correction_maximum(m, (float)d));
  DLB_TRY(s.expect("|END| NORMALIZATION PARAMETERS |END|"));
  DLB_TRY(skip_section("LOSS PARAMETERS", {"loss_train", "loss_valid", "loss_testg"}));
  DLB_TRY(s.expect("|===| ACCURANCY PARAMETERS |===|"));
  DLB_TRY(s.real("acc_var", &d));
  DLB_TRY(dlb_model_set_accu_var(m, (float)d));
  for (const char *k : {"acc_train", "acc_valid", "acc_testg"}) DLB_TRY(s.real(k, &d));
  DLB_TRY(s.expect("|END| ACCURANCY PARAMETERS |END|"));
  DLB_TRY(s.expect("|===| COMPUTATION PARAMETERS |===|"));
  DLB_TRY(s.real("use_cu", &d));
  DLB_TRY(s.real("use_mp", &d));
  DLB_TRY(s.real("pct_threads", &d));
  size_t max_batch;
  DLB_TRY(s.count("maximum_batch_size", &max_batch));
  DLB_TRY(dlb_model_set_max_batch_size(m, max_batch));
  DLB_TRY(s.expect("|END| COMPUTATION PARAMETERS |END|"));

  // Weights, biases, scales, shifts and running averages.
  DLB_REQUIRE(m->total_parameters == 0 || dlb_model_get_size(m, "total_parameters") == total_parameters,
              "load: the layers of the file give another parameter count than its header");
  std::vector<float> params(total_parameters, 0.f);
  DLB_TRY(dlb_model_get_array(m, "parameters", params.data(), total_parameters));
  for (size_t i = 0; i < n_layers; ++i) {
    for (const auto &w : L[i].weights) {
      DLB_REQUIRE(w.first < total_parameters, "load: weight index out of range");
      params[w.first] = w.second;
    }
    if (L[i].norm == DLB_NORM_NONE) continue;
    const LayerRT &l = m->layers[i];
    DLB_REQUIRE(L[i].scale.size() == l.norm_units, "load: a layer's normalized units do not match its shape");
    for (size_t k = 0; k < L[i].scale.size(); ++k) {
      params[gamma_at(m, l) + k] = L[i].scale[k];
      params[beta_at(m, l) + k] = L[i].shift[k];
    }
  }
  DLB_TRY(dlb_model_set_array(m, "parameters", params.data(), total_parameters));
  for (size_t i = 0; i < n_layers; ++i) {
    if (L[i].norm == DLB_NORM_NONE) continue;
    DLB_TRY(dlb_model_set_layer_norm(m, i, "mean_average", L[i].mean_avg.data(), L[i].mean_avg.size()));
    DLB_TRY(dlb_model_set_layer_norm(m, i, "variance_average", L[i].sigma_avg.data(), L[i].sigma_avg.size()));
  }
  return DLB_OK;
}

}  // extern "C"
