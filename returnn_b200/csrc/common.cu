// Error string storage shared by all entry points.
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

static thread_local char g_err[512] = {0};

void rb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

RB_EXPORT const char* rb200_last_error() { return g_err; }

RB_EXPORT int rb200_version() { return 1; }

// programmatic dependent launch on/off (see common.cuh), read once from RETURNN_B200_PDL
bool rb_pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("RETURNN_B200_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}
