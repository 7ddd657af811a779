/* Test infrastructure, not product code.
 *
 * Hook macros that oracle/dropin_patch.py inserts at the top of the reference's
 * step entry points (inside member functions of DL::v1::Model).  While the
 * model's b200_on switch is set, the call is served by libdlb200 and the
 * reference's own OpenMP code below the hook is skipped.  The entry points are
 * entered by every thread of one OpenMP team (drivers/driver.cpp L:241-257); the
 * library takes one caller per context, so the team's first thread makes the call.
 */
#pragma once
#include <stddef.h>

namespace DL::v1 {
class Model;
}
namespace dlb_dropin {
void forward(DL::v1::Model *m, size_t rows, float const *const *Xm);
void error(DL::v1::Model *m, size_t rows, float const *const *Ym);
void backward(DL::v1::Model *m, size_t rows);
void derivatives(DL::v1::Model *m, size_t rows);
void merge(DL::v1::Model *m);
void update(DL::v1::Model *m, size_t rows, size_t training_size);
double loss(DL::v1::Model const *m);
void reset_loss(DL::v1::Model *m);
bool first_thread();
}  // namespace dlb_dropin

#define DLB_DROPIN_FORWARD(rows, Xm) \
  if (this->b200_on) { if (dlb_dropin::first_thread()) dlb_dropin::forward(this, rows, Xm); return; }
#define DLB_DROPIN_ERROR(rows, Ym) \
  if (this->b200_on) { if (dlb_dropin::first_thread()) dlb_dropin::error(this, rows, Ym); return; }
#define DLB_DROPIN_BACKWARD(rows) \
  if (this->b200_on) { if (dlb_dropin::first_thread()) dlb_dropin::backward(this, rows); return; }
#define DLB_DROPIN_DERIVATIVES(rows) \
  if (this->b200_on) { if (dlb_dropin::first_thread()) dlb_dropin::derivatives(this, rows); return; }
#define DLB_DROPIN_MERGE() \
  if (this->b200_on) { dlb_dropin::merge(this); return; }
#define DLB_DROPIN_UPDATE(rows, training_size) \
  if (this->b200_on) { dlb_dropin::update(this, rows, training_size); return; }
#define DLB_DROPIN_GET_LOSS(env) \
  if (this->b200_on && env == ENV::NONE) return dlb_dropin::loss(this);
#define DLB_DROPIN_RESET_LOSS() \
  if (this->b200_on) dlb_dropin::reset_loss(this);
