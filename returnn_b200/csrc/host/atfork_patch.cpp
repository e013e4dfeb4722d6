// LD_PRELOAD library that turns pthread_atfork / __register_atfork into no-ops and runs fork() without the registered handlers.
// Some libraries (OpenBLAS, CUDA-aware MPI builds) register atfork handlers that dead-lock or crash in a forked child that only
// wants to exec; with this library preloaded (config option patch_atfork) they never run. Counterpart of the C snippet in the
// reference (returnn/util/basic.py:3895-3950).
#include <sys/syscall.h>
#include <sys/types.h>
#include <unistd.h>

extern "C" {
__attribute__((visibility("default"))) int pthread_atfork(void (*)(void), void (*)(void), void (*)(void)) { return 0; }
__attribute__((visibility("default"))) int __register_atfork(void (*)(void), void (*)(void), void (*)(void), void*) { return 0; }
__attribute__((visibility("default"))) pid_t fork(void) { return (pid_t)syscall(SYS_fork); }
}
