// Checkpoint directories in the reference's layout, with rotation:
//
//   <dir>/checkpoint                 "model_checkpoint_path: ckpt-<step>"
//   <dir>/ckpt-<step>/model.net      Model::save_params
//   <dir>/ckpt-<step>/model.nn       Model::save_spec_params
//   <dir>/ckpt-<step>/model.opt      optimizer moments (this library's addition)
//
// ref: DL::Checkpointer (nn/checkpointer.cpp L:41-160: load, save, rotate,
// save_model_checkpoint_path, read_model_checkpoint_path) and
// CheckpointerInterval::operator() (L:223-250).  The reference's format has no
// optimizer state; model.opt is a binary side file that the reference ignores:
//   char magic[8] "DLBOPT1", u64 P, i32 optimizer, f32 optimizer_time_step,
//   f32 adam_previous_beta2, f32 epoch_time_step, then first[P], second[P],
//   second_hat[P] as raw floats.
// Host code only.
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <filesystem>
#include <fstream>
#include <string>
#include <vector>

#include "common.cuh"
#include "model.cuh"

namespace fs = std::filesystem;
using namespace dlb;

struct dlb_checkpointer {
  dlb_model *model = nullptr;
  std::string dir;
  int max_to_keep = 1;
  int interval = 1;
  int next_step = 0;  // CheckpointerInterval::next_step
};

namespace {

const char MAGIC[8] = {'D', 'L', 'B', 'O', 'P', 'T', '1', '\0'};

struct OptHeader {
  char magic[8];
  uint64_t parameters;
  int32_t optimizer;
  float optimizer_time_step, adam_previous_beta2, epoch_time_step;
};

dlb_status save_moments(dlb_model *m, const std::string &path) {
  const size_t P = m->total_parameters;
  OptHeader h{};
  memcpy(h.magic, MAGIC, 8);
  h.parameters = P;
  h.optimizer = m->optimizer;
  h.optimizer_time_step = m->hp.optimizer_time_step;
  h.adam_previous_beta2 = m->hp.adam_previous_beta2;
  h.epoch_time_step = m->hp.epoch_time_step;
  std::ofstream f(path, std::ios::binary);
  if (!f) {
    set_error("checkpointer: cannot write %s", path.c_str());
    return DLB_ERR_INVALID;
  }
  f.write(reinterpret_cast<const char *>(&h), sizeof(h));
  std::vector<float> buf(P);
  for (const char *name : {"first_moment", "second_moment", "second_moment_hat"}) {
    DLB_TRY(dlb_model_get_array(m, name, buf.data(), P));
    f.write(reinterpret_cast<const char *>(buf.data()), (std::streamsize)(P * sizeof(float)));
  }
  f.close();
  if (!f) {
    set_error("checkpointer: short write to %s", path.c_str());
    return DLB_ERR_INVALID;
  }
  return DLB_OK;
}

// Moments of a model that has just been loaded from the same directory; a
// missing file leaves them at zero (a checkpoint written by the reference).
dlb_status load_moments(dlb_model *m, const std::string &path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return DLB_OK;
  OptHeader h{};
  f.read(reinterpret_cast<char *>(&h), sizeof(h));
  if (!f || memcmp(h.magic, MAGIC, 8) != 0 || h.parameters != m->total_parameters) {
    set_error("checkpointer: %s does not belong to this model", path.c_str());
    return DLB_ERR_INVALID;
  }
  const size_t P = m->total_parameters;
  std::vector<float> buf(P);
  for (const char *name : {"first_moment", "second_moment", "second_moment_hat"}) {
    f.read(reinterpret_cast<char *>(buf.data()), (std::streamsize)(P * sizeof(float)));
    if (!f) {
      set_error("checkpointer: %s is truncated", path.c_str());
      return DLB_ERR_INVALID;
    }
    DLB_TRY(dlb_model_set_array(m, name, buf.data(), P));
  }
  m->hp.optimizer_time_step = h.optimizer_time_step;
  m->hp.adam_previous_beta2 = h.adam_previous_beta2;
  m->hp.epoch_time_step = h.epoch_time_step;
  return DLB_OK;
}

// Checkpointer::rotate (nn/checkpointer.cpp L:136-160): the newest max_to_keep
// checkpoint directories by time of last write stay, the others are removed.
// Only directories named ckpt-* count here; the reference walks every directory
// under <dir>.
void rotate(const dlb_checkpointer *c) {
  std::vector<std::pair<fs::file_time_type, fs::path>> found;
  std::error_code ec;
  for (const auto &entry : fs::directory_iterator(c->dir, ec)) {
    if (!entry.is_directory(ec)) continue;
    if (entry.path().filename().string().rfind("ckpt-", 0) != 0) continue;
    found.emplace_back(entry.last_write_time(ec), entry.path());
  }
  if ((int)found.size() <= c->max_to_keep) return;
  std::sort(found.begin(), found.end(), [](const auto &a, const auto &b) { return a.first > b.first; });
  for (size_t i = (size_t)c->max_to_keep; i < found.size(); ++i) fs::remove_all(found[i].second, ec);
}

}  // namespace

extern "C" {

dlb_status dlb_checkpointer_create(dlb_checkpointer **out, dlb_model *model, const char *ckpt_dir,
                                   int max_to_keep, int interval) {
  DLB_REQUIRE(out && model && ckpt_dir && max_to_keep >= 1 && interval >= 1, "dlb_checkpointer_create");
  *out = new dlb_checkpointer;
  (*out)->model = model;
  (*out)->dir = ckpt_dir;
  (*out)->max_to_keep = max_to_keep;
  (*out)->interval = interval;
  return DLB_OK;
}

dlb_status dlb_checkpointer_destroy(dlb_checkpointer *c) {
  delete c;
  return DLB_OK;
}

// ref: Checkpointer::save (nn/checkpointer.cpp L:94-130).
dlb_status dlb_checkpointer_save(dlb_checkpointer *c, int step_train) {
  DLB_REQUIRE(c && step_train >= 0, "dlb_checkpointer_save");
  const std::string name = "ckpt-" + std::to_string(step_train);
  const fs::path at = fs::path(c->dir) / name;
  std::error_code ec;
  fs::create_directories(at, ec);
  if (ec) {
    set_error("checkpointer: cannot create %s: %s", at.string().c_str(), ec.message().c_str());
    return DLB_ERR_INVALID;
  }
  DLB_TRY(dlb_model_save_params(c->model, (at / "model.net").string().c_str()));
  DLB_TRY(dlb_model_save_spec_params(c->model, (at / "model.nn").string().c_str()));
  DLB_TRY(save_moments(c->model, (at / "model.opt").string()));
  // Checkpointer::save_model_checkpoint_path (L:162-182): one line, no line end.
  std::ofstream f(fs::path(c->dir) / "checkpoint", std::ios::binary);
  f << "model_checkpoint_path: " << name;
  f.close();
  if (!f) {
    set_error("checkpointer: cannot write %s/checkpoint", c->dir.c_str());
    return DLB_ERR_INVALID;
  }
  rotate(c);
  return DLB_OK;
}

// ref: CheckpointerInterval::operator() (nn/checkpointer.cpp L:230-250): saves
// when forced, or when step g has reached next_step and the run's metrics are at
// their best so far (is_top; pass 1 where no such record is kept), then moves
// next_step to g + interval.
dlb_status dlb_checkpointer_step(dlb_checkpointer *c, int g, int step_train, int is_top, int force, int *saved) {
  DLB_REQUIRE(c && saved, "dlb_checkpointer_step");
  *saved = 0;
  if (force || (g >= c->next_step && is_top)) {
    c->next_step = g + c->interval;
    DLB_TRY(dlb_checkpointer_save(c, step_train));
    *saved = 1;
  }
  return DLB_OK;
}

// ref: Checkpointer::load (nn/checkpointer.cpp L:51-92) with
// read_model_checkpoint_path (L:184-221).  The model must not have been compiled
// (dlb_model_load builds it from the files).  *found = 0 and DLB_OK when the
// directory holds no checkpoint.
dlb_status dlb_checkpointer_load(dlb_checkpointer *c, int *found) {
  DLB_REQUIRE(c && found, "dlb_checkpointer_load");
  *found = 0;
  std::ifstream f(fs::path(c->dir) / "checkpoint", std::ios::binary);
  if (!f) return DLB_OK;
  std::string key, name;
  f >> key >> name;
  if (key != "model_checkpoint_path:" || name.empty()) {
    set_error("checkpointer: %s/checkpoint is not a checkpoint record", c->dir.c_str());
    return DLB_ERR_INVALID;
  }
  const fs::path at = fs::path(c->dir) / name;
  std::error_code ec;
  if (!fs::exists(at / "model.net", ec) || !fs::exists(at / "model.nn", ec)) return DLB_OK;
  DLB_TRY(dlb_model_load(c->model, (at / "model.net").string().c_str(), (at / "model.nn").string().c_str()));
  DLB_TRY(load_moments(c->model, (at / "model.opt").string()));
  *found = 1;
  return DLB_OK;
}

}  // extern "C"
