// Host-only check of the library's C++ that runs on the CPU: the per-thread error channel (formatting, truncation at
// the buffer's end, one message per thread) and the small queries beside it.  Built by the test suite with
// -fsanitize=address,undefined and run as it is; exit code 0 when every case passes, one line per failure otherwise.
// The reference keeps the same channel in TSGgml_GetLastError (TensorSharp.GGML.Native/ggml_ops_core.cpp:1117).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../common.cuh"

extern "C" int tsb_abi_version();
bool tsb_pdl_enabled();

static int failures = 0;
#define EXPECT(cond)                                                     \
    do {                                                                 \
        if (!(cond)) {                                                   \
            std::printf("FAIL line %d: %s\n", __LINE__, #cond);         \
            ++failures;                                                  \
        }                                                                \
    } while (0)

static int checked(int v) {
    TSB_CHECK_ARG(v >= 0, "value %d is negative (%s)", v, "checked");
    return TSB_OK;
}

int main() {
    EXPECT(tsb_abi_version() == 1);
    EXPECT(std::strlen(tsb_last_error()) == 0);
    EXPECT(checked(3) == TSB_OK);
    EXPECT(checked(-7) == TSB_ERR_ARG);
    EXPECT(std::strcmp(tsb_last_error(), "value -7 is negative (checked)") == 0);
    // a message longer than the buffer is cut, not written past the end
    const std::string big(5000, 'x');
    tsb_set_error("%s", big.c_str());
    const size_t n = std::strlen(tsb_last_error());
    EXPECT(n > 0 && n < 5000);
    EXPECT(tsb_last_error()[n - 1] == 'x');
    // every thread has its own message
    std::vector<std::thread> ts;
    std::vector<int> ok(8, 0);
    for (int t = 0; t < 8; ++t) {
        ts.emplace_back([t, &ok]() {
            bool good = std::strlen(tsb_last_error()) == 0;          // a fresh thread starts empty
            for (int i = 0; i < 200; ++i) {
                tsb_set_error("thread %d message %d", t, i);
                char want[64];
                std::snprintf(want, sizeof(want), "thread %d message %d", t, i);
                good = good && std::strcmp(tsb_last_error(), want) == 0;
            }
            ok[t] = good ? 1 : 0;
        });
    }
    for (auto& th : ts) th.join();
    for (int t = 0; t < 8; ++t) EXPECT(ok[t] == 1);
    EXPECT(std::strlen(tsb_last_error()) == n);                       // the main thread's message is untouched
    const bool want_pdl = std::getenv("TSB_DISABLE_PDL") == nullptr;
    EXPECT(tsb_pdl_enabled() == want_pdl);
    if (failures == 0) std::printf("OK\n");
    return failures == 0 ? 0 : 1;
}
