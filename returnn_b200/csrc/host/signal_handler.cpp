// Crash signal handler: on SIGSEGV / SIGBUS / SIGILL / SIGABRT / SIGFPE / SIGUSR1 write the C backtrace to stderr (async-signal-safe
// backtrace_symbols_fd), then restore the previous disposition and re-raise, so that Python's faulthandler and the core dump
// still happen. Counterpart of the C helper in the reference (returnn/util/debug.py:283-345).
#include <execinfo.h>
#include <signal.h>
#include <string.h>
#include <unistd.h>

namespace {
struct sigaction g_old[65];

void write_str(const char* s) {
  ssize_t r = write(STDERR_FILENO, s, strlen(s));
  (void)r;
}

void handler(int sig) {
  write_str("\nSignal handler: signal ");
  char buf[16];
  int n = sig, i = 15;
  buf[i] = 0;
  do {
    buf[--i] = (char)('0' + n % 10);
    n /= 10;
  } while (n && i > 0);
  write_str(buf + i);
  write_str(", C backtrace:\n");
  void* frames[64];
  int cnt = backtrace(frames, 64);
  backtrace_symbols_fd(frames, cnt, STDERR_FILENO);
  if (sig == SIGUSR1) return;  // informational only
  sigaction(sig, &g_old[sig], nullptr);
  raise(sig);
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int rb200_install_signal_handler(int sig) {
  if (sig <= 0 || sig >= 65) return -1;
  struct sigaction sa;
  memset(&sa, 0, sizeof(sa));
  sa.sa_handler = handler;
  sigemptyset(&sa.sa_mask);
  sa.sa_flags = SA_NODEFER;
  return sigaction(sig, &sa, &g_old[sig]);
}

extern "C" __attribute__((visibility("default"))) int rb200_install_default_signal_handlers() {
  const int sigs[] = {SIGSEGV, SIGBUS, SIGILL, SIGABRT, SIGFPE, SIGUSR1};
  int rc = 0;
  for (int s : sigs) rc |= rb200_install_signal_handler(s);
  return rc;
}
