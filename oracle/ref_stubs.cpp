/* Test infrastructure, not product code.
 *
 * Aborting definitions for the handful of reference symbols whose own source
 * files need Boost, Eigen or libsystemd and are therefore left out of
 * oracle/_ref/libdlref.so.  They are referenced only from the reference's
 * save/load, console and LSUV/orthogonal-init code, none of which the
 * fully-connected training step reaches; reaching one is a harness bug.
 */
#include "pch.hpp"

#include "deep-learning/io/file.hpp"
#include "deep-learning/v1/data/datasets.hpp"
#include "deep-learning/v1/learner/model.hpp"

#include <cstdio>
#include <cstdlib>

[[noreturn]] static void off_path(const char *what) {
  std::fprintf(stderr, "oracle/_ref: %s is not part of the oracle build\n",
               what);
  std::abort();
}

namespace DL::File {
bool create_temp_file(std::wstring const &) { return true; }
bool delete_temp_file(std::wstring const &) { return true; }
bool recover_temp_file(std::wstring const &) { return true; }
bool path_exist(std::wstring const &path) {
  std::string narrow(path.begin(), path.end());
  if (FILE *f = std::fopen(narrow.c_str(), "rb")) {
    std::fclose(f);
    return true;
  }
  return false;
}

template <typename T>
bool read_stream_block_n_parse(wchar_t *&, wchar_t *&, size_t &, size_t const,
                               size_t const, T &, std::vector<wchar_t> &,
                               std::wifstream &, wchar_t const) {
  off_path("File::read_stream_block_n_parse");
}
template bool read_stream_block_n_parse<double>(
    wchar_t *&, wchar_t *&, size_t &, size_t const, size_t const, double &,
    std::vector<wchar_t> &, std::wifstream &, wchar_t const);
template bool read_stream_block_n_parse<size_t>(
    wchar_t *&, wchar_t *&, size_t &, size_t const, size_t const, size_t &,
    std::vector<wchar_t> &, std::wifstream &, wchar_t const);
}  // namespace DL::File

namespace DL::v1 {
Datasets::Datasets(void) { off_path("Datasets::Datasets"); }
Datasets::~Datasets(void) {}
bool Datasets::Get__Dataset_In_Equal_Less_Holdout_Accepted(void) const {
  off_path("Datasets::Get__Dataset_In_Equal_Less_Holdout_Accepted");
}
double Datasets::Get__Minimum_Loss_Holdout_Accepted(void) const {
  off_path("Datasets::Get__Minimum_Loss_Holdout_Accepted");
}
ENV::TYPE Datasets::Get__Type_Dataset_Evaluation(void) const {
  off_path("Datasets::Get__Type_Dataset_Evaluation");
}
double Datasets::Type_Testing(ENV::TYPE const, Model *const) {
  off_path("Datasets::Type_Testing");
}
bool Datasets::Use__Metric_Loss(void) const {
  off_path("Datasets::Use__Metric_Loss");
}
bool Datasets::reference(Datasets *const) { off_path("Datasets::reference"); }
bool Datasets::Deallocate(void) { off_path("Datasets::Deallocate"); }
double Datasets::train(Model *const) { off_path("Datasets::train"); }
double Datasets::evaluate(Model *const) { off_path("Datasets::evaluate"); }

void Model::layers_initialize_orthogonal(bool const, real const) {
  off_path("Model::layers_initialize_orthogonal");
}
}  // namespace DL::v1
