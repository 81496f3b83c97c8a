// Last-error string shared by every exported entry point (thread-local).
// Reference counterpart: TSGgml_GetLastError (TensorSharp.GGML.Native/ggml_ops_core.cpp:1117).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include "common.cuh"

static thread_local char g_err[1024] = "";

void tsb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

extern "C" const char* tsb_last_error() { return g_err; }

extern "C" int tsb_abi_version() { return 1; }

// Programmatic dependent launch is on unless TSB_DISABLE_PDL is set in the environment.
bool tsb_pdl_enabled() {
    static const bool on = (std::getenv("TSB_DISABLE_PDL") == nullptr);
    return on;
}
