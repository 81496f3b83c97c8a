// Stand-alone check of the library's C interface, without Python: quantised row gather and the quantised
// matrix-vector product against a host restatement, plus the error channel.  Links libtsb200.so.
//
//     native_check [rows] [k]        exit code 0 when every case passes; one line per case on stdout
//
// Plays the part of the reference's native test executables (TensorSharp.GGML.Native/tests/get_rows_quant_test.cpp,
// addmm_vector_test.cpp).  Weights are made directly in the device layout of Q8_0 (int8 values [N][K] and one half
// scale per 32 values [N][K/32]), so the program needs no GGUF file.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

extern "C" {
int tsb_abi_version();
const char* tsb_last_error();
int tsb_quantize_q8(const void* x, int x_is_f32, void* xq, void* xds, long rows, int K, void* stream);
int tsb_gemv(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K, const void* xq,
             const void* xds, const void* xb, void* out, const float* bias, const void* residual, const int* ids,
             const float* row_scale, int M, int problems, int x_div, int out_f32, int act, void* stream);
int tsb_gather_rows(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K, const int* ids,
                    long n_rows, float scale, void* out, int out_f32, void* stream);
}

static const int TYPE_Q8_0 = 8;          // GGML type number

#define CUDA_OK(call)                                                                              \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            std::printf("FAIL cuda %s at line %d: %s\n", #call, __LINE__, cudaGetErrorString(e_)); \
            return 2;                                                                              \
        }                                                                                          \
    } while (0)

template <typename T>
struct DeviceBuf {
    T* p = nullptr;
    size_t n = 0;
    explicit DeviceBuf(size_t count) : n(count) { cudaMalloc(&p, count * sizeof(T)); }
    ~DeviceBuf() { cudaFree(p); }
    bool up(const std::vector<T>& h) { return cudaMemcpy(p, h.data(), n * sizeof(T), cudaMemcpyHostToDevice) == cudaSuccess; }
    bool down(std::vector<T>& h) const {
        h.resize(n);
        return cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost) == cudaSuccess;
    }
};

struct Q8Weight {
    int N, K;
    std::vector<int8_t> q;       // [N][K]
    std::vector<__half> d;       // [N][K/32]
    float at(int r, int c) const { return (float)q[(size_t)r * K + c] * __half2float(d[(size_t)r * (K / 32) + c / 32]); }
};

static Q8Weight make_weight(int N, int K, unsigned seed) {
    Q8Weight w{N, K, {}, {}};
    std::mt19937 rng(seed);
    std::uniform_int_distribution<int> qv(-127, 127);
    std::uniform_real_distribution<float> dv(0.001f, 0.02f);
    w.q.resize((size_t)N * K);
    w.d.resize((size_t)N * (K / 32));
    for (auto& v : w.q) v = (int8_t)qv(rng);
    for (auto& v : w.d) v = __float2half(dv(rng));
    return w;
}

static int g_failed = 0;

static void report(const char* name, bool ok, double err, double tol) {
    std::printf("%s %s max_err=%.3g tol=%.3g\n", ok ? "PASS" : "FAIL", name, err, tol);
    if (!ok) ++g_failed;
}

// Rows picked by index, dequantised and scaled: exact in f32 (one int8 times one half times the scale).
static int check_gather(const Q8Weight& w, int n_pick) {
    std::mt19937 rng(7);
    std::uniform_int_distribution<int> pick(0, w.N - 1);
    std::vector<int> ids(n_pick);
    for (auto& i : ids) i = pick(rng);
    const float scale = 1.5f;
    DeviceBuf<int8_t> dq(w.q.size());
    DeviceBuf<__half> dd(w.d.size());
    DeviceBuf<int> di(ids.size());
    DeviceBuf<float> dout((size_t)n_pick * w.K);
    if (!dq.up(w.q) || !dd.up(w.d) || !di.up(ids)) return 2;
    if (tsb_gather_rows(dq.p, dd.p, nullptr, nullptr, TYPE_Q8_0, w.N, w.K, di.p, n_pick, scale, dout.p, 1, nullptr) != 0) {
        std::printf("FAIL gather_rows_q8_0 call: %s\n", tsb_last_error());
        ++g_failed;
        return 0;
    }
    CUDA_OK(cudaDeviceSynchronize());
    std::vector<float> out;
    if (!dout.down(out)) return 2;
    double worst = 0.0;
    for (int r = 0; r < n_pick; ++r)
        for (int c = 0; c < w.K; ++c)
            worst = std::fmax(worst, std::fabs((double)out[(size_t)r * w.K + c] - (double)w.at(ids[r], c) * scale));
    report("gather_rows_q8_0", worst <= 1e-5, worst, 1e-5);
    return 0;
}

// y[m][n] = sum_k W[n][k] x[m][k] with the activations quantised to int8 groups by the library itself.  Two checks:
// against the same integer arithmetic restated on the host (tight), and against the float product (the quantisation
// error of 8-bit activations, loose).
static int check_gemv(const Q8Weight& w, int M) {
    std::mt19937 rng(11 + M);
    std::normal_distribution<float> nv(0.f, 1.f);
    std::vector<float> x((size_t)M * w.K);
    for (auto& v : x) v = nv(rng);
    const int kb = w.K / 32;
    DeviceBuf<int8_t> dq(w.q.size());
    DeviceBuf<__half> dd(w.d.size());
    DeviceBuf<float> dx(x.size());
    DeviceBuf<int8_t> dxq(x.size());
    DeviceBuf<float2> dxds((size_t)M * kb);
    DeviceBuf<float> dout((size_t)M * w.N);
    if (!dq.up(w.q) || !dd.up(w.d) || !dx.up(x)) return 2;
    char name[64];
    std::snprintf(name, sizeof(name), "gemv_q8_0_m%d", M);
    if (tsb_quantize_q8(dx.p, 1, dxq.p, dxds.p, M, w.K, nullptr) != 0 ||
        tsb_gemv(dq.p, dd.p, nullptr, nullptr, TYPE_Q8_0, w.N, w.K, dxq.p, dxds.p, nullptr, dout.p, nullptr, nullptr, nullptr,
                 nullptr, M, 1, 1, 1, 0, nullptr) != 0) {
        std::printf("FAIL %s call: %s\n", name, tsb_last_error());
        ++g_failed;
        return 0;
    }
    CUDA_OK(cudaDeviceSynchronize());
    std::vector<float> out;
    std::vector<int8_t> xq;
    std::vector<float2> xds;
    if (!dout.down(out) || !dxq.down(xq) || !dxds.down(xds)) return 2;
    double worst_int = 0.0, worst_float = 0.0, scale_ref = 0.0;
    for (int m = 0; m < M; ++m) {
        for (int n = 0; n < w.N; ++n) {
            double acc_int = 0.0, acc_float = 0.0;
            for (int g = 0; g < kb; ++g) {
                long dot = 0;
                for (int j = 0; j < 32; ++j) {
                    const size_t k = (size_t)g * 32 + j;
                    dot += (long)w.q[(size_t)n * w.K + k] * (long)xq[(size_t)m * w.K + k];
                    acc_float += (double)w.at(n, (int)k) * (double)x[(size_t)m * w.K + k];
                }
                acc_int += (double)__half2float(w.d[(size_t)n * kb + g]) * (double)xds[(size_t)m * kb + g].x * (double)dot;
            }
            const double got = out[(size_t)m * w.N + n];
            worst_int = std::fmax(worst_int, std::fabs(got - acc_int));
            worst_float = std::fmax(worst_float, std::fabs(got - acc_float));
            scale_ref = std::fmax(scale_ref, std::fabs(acc_float));
        }
    }
    report(name, worst_int <= 1e-3 * std::fmax(1.0, scale_ref), worst_int, 1e-3 * std::fmax(1.0, scale_ref));
    std::snprintf(name, sizeof(name), "gemv_q8_0_m%d_vs_float", M);
    report(name, worst_float <= 3e-2 * std::fmax(1.0, scale_ref), worst_float, 3e-2 * std::fmax(1.0, scale_ref));
    return 0;
}

// A call with a shape the kernels cannot take returns a status and leaves a message; nothing is launched.
static void check_error_channel(const Q8Weight& w) {
    const int rc = tsb_gemv(nullptr, nullptr, nullptr, nullptr, TYPE_Q8_0, w.N, 33, nullptr, nullptr, nullptr, nullptr, nullptr,
                            nullptr, nullptr, nullptr, 1, 1, 1, 1, 0, nullptr);
    const char* msg = tsb_last_error();
    const bool ok = rc != 0 && msg != nullptr && std::strlen(msg) > 0;
    std::printf("%s error_channel rc=%d message=\"%s\"\n", ok ? "PASS" : "FAIL", rc, msg ? msg : "");
    if (!ok) ++g_failed;
}

int main(int argc, char** argv) {
    const int N = argc > 1 ? std::atoi(argv[1]) : 512;
    const int K = argc > 2 ? std::atoi(argv[2]) : 1024;
    if (N <= 0 || K <= 0 || K % 32 != 0) {
        std::printf("usage: native_check [rows > 0] [k: a multiple of 32]\n");
        return 2;
    }
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
        std::printf("SKIP no CUDA device\n");
        return 77;
    }
    std::printf("abi_version %d rows %d k %d\n", tsb_abi_version(), N, K);
    const Q8Weight w = make_weight(N, K, 3);
    check_error_channel(w);
    if (int rc = check_gather(w, 37)) return rc;
    for (int M : {1, 4, 16})
        if (int rc = check_gemv(w, M)) return rc;
    std::printf("%s\n", g_failed ? "FAILED" : "OK");
    return g_failed ? 1 : 0;
}
