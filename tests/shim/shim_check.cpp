// A host program written against the reference's own names (xinfer::ops::..., xinfer::core::DeviceContext,
// xinfer::core::DeviceArena) through include/xinfer_b200_ops.hpp, built with plain g++ and linked to
// libxinfer_b200.so: the compiled proof that the shim makes callers of src/ops/linear.h:30-139,
// src/ops/sampling.h:11-49 and src/core/arena.h:14-66 build with only the queue type changed.  The cases are
// the reference tests' own (tests/test_ops_oracle.cpp:290-792, 911-947; tests/test_speculative_mtp.cpp:83-189;
// tests/test_core_device.cpp arena contract), with their inline fp64 expectations recomputed here.
//
//   shim_check            runs everything on the current CUDA device, prints one line per case, exits 0 on success
//   shim_check --list     prints the case names (no device needed)
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "xinfer_b200_ops.hpp"

using namespace xinfer;
using half_t = _Float16;  // the fp16 storage type on the host side

namespace {

int g_failed = 0;
void report(const char* name, bool ok, double value) {
    std::printf("%-34s %s  (%.3g)\n", name, ok ? "ok" : "FAILED", value);
    if (!ok) ++g_failed;
}

std::vector<uint8_t> fill_w(size_t n, int a, int b) {
    std::vector<uint8_t> w(n);
    for (size_t i = 0; i < n; ++i) w[i] = static_cast<uint8_t>(((i + a) & 0xF) | (((i + b) & 0xF) << 4));
    return w;
}
std::vector<half_t> fill_s(size_t n, float base = 0.015f, int shift = 0) {
    std::vector<half_t> s(n);
    for (size_t i = 0; i < n; ++i) s[i] = static_cast<half_t>(base + static_cast<float>((i + shift) % 10) * 0.001f);
    return s;
}
inline int nib(const std::vector<uint8_t>& w, size_t row_bytes, size_t n, size_t k) {
    const uint8_t b = w[n * row_bytes + k / 2];
    const int v = (k & 1) ? (b >> 4) : (b & 0xF);
    return v >= 8 ? v - 16 : v;
}
// per-group fp64 dot times the group's scale, summed in fp64: the reference tests' inline expectation
double dot_row(const float* x, const std::vector<uint8_t>& w, const std::vector<half_t>& s, size_t n, size_t K) {
    double acc = 0.0;
    for (size_t g = 0; g < K / 128; ++g) {
        double d = 0.0;
        for (size_t k = g * 128; k < (g + 1) * 128; ++k) d += static_cast<double>(x[k]) * nib(w, K / 2, n, k);
        acc += d * static_cast<double>(static_cast<float>(s[n * (K / 128) + g]));
    }
    return acc;
}

template <typename T>
T* to_device(core::DeviceContext& ctx, const std::vector<T>& v) {
    T* d = static_cast<T*>(ctx.allocate_device(v.size() * sizeof(T)));
    ctx.copy_host_to_device(d, v.data(), v.size() * sizeof(T));
    return d;
}

void linear_cases(core::DeviceContext& ctx) {
    std::mt19937 rng(46);
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    {   // fp32 in / fp32 out, M=2 K=5120 N=2048, max-abs 1e-4
        const size_t M = 2, K = 5120, N = 2048;
        std::vector<float> X(M * K);
        for (auto& v : X) v = dist(rng);
        auto W = fill_w(N * K / 2, 3, 7);
        auto S = fill_s(N * (K / 128));
        float* dX = to_device(ctx, X);
        uint8_t* dW = to_device(ctx, W);
        half_t* dS = to_device(ctx, S);
        float* dY = static_cast<float*>(ctx.allocate_device(M * N * sizeof(float)));
        ops::linear_int4(ctx.queue(), dY, dX, dW, dS, nullptr, M, N, K, 128);
        std::vector<float> Y(M * N);
        ctx.copy_device_to_host(Y.data(), dY, Y.size() * sizeof(float));
        double worst = 0;
        for (size_t m = 0; m < M; ++m)
            for (size_t n = 0; n < N; ++n) worst = std::fmax(worst, std::fabs(Y[m * N + n] - dot_row(&X[m * K], W, S, n, K)));
        report("linear_int4 f32 M2 K5120 N2048", worst <= 1e-4, worst);
        ctx.free_device(dX); ctx.free_device(dW); ctx.free_device(dS); ctx.free_device(dY);
    }
    {   // the split-K shape M=1 N=48, max-abs 1e-3
        const size_t K = 5120, N = 48;
        std::vector<float> X(K);
        for (auto& v : X) v = dist(rng);
        auto W = fill_w(N * K / 2, 5, 11);
        auto S = fill_s(N * (K / 128));
        float* dX = to_device(ctx, X);
        uint8_t* dW = to_device(ctx, W);
        half_t* dS = to_device(ctx, S);
        float* dY = static_cast<float*>(ctx.allocate_device(N * sizeof(float)));
        ops::linear_int4(ctx.queue(), dY, dX, dW, dS, nullptr, 1, N, K);
        std::vector<float> Y(N);
        ctx.copy_device_to_host(Y.data(), dY, Y.size() * sizeof(float));
        double worst = 0;
        for (size_t n = 0; n < N; ++n) worst = std::fmax(worst, std::fabs(Y[n] - dot_row(X.data(), W, S, n, K)));
        report("linear_int4 split-K N48", worst <= 1e-3, worst);
        ctx.free_device(dX); ctx.free_device(dW); ctx.free_device(dS); ctx.free_device(dY);
    }
    {   // four fused projections N = {128, 64, 48, 48}, K = 512, and num_descs outside [1,4] as a silent no-op
        const size_t K = 512;
        const size_t Ns[4] = {128, 64, 48, 48};
        std::vector<float> X(K);
        for (auto& v : X) v = dist(rng);
        float* dX = to_device(ctx, X);
        ops::FusedProjectionDescFP32 d[4];
        std::vector<std::vector<uint8_t>> Ws;
        std::vector<std::vector<half_t>> Ss;
        for (int p = 0; p < 4; ++p) {
            Ws.push_back(fill_w(Ns[p] * K / 2, p + 3, p + 7));
            Ss.push_back(fill_s(Ns[p] * (K / 128), 0.015f, p));
            d[p].W_int4 = to_device(ctx, Ws[p]);
            d[p].scales = to_device(ctx, Ss[p]);
            d[p].bias = nullptr;
            d[p].N = static_cast<int64_t>(Ns[p]);
            d[p].Y = ctx.allocate_device(Ns[p] * sizeof(float));
        }
        ops::linear_int4_fused(ctx.queue(), dX, d, 4, 1, K);
        ops::linear_int4_fused(ctx.queue(), dX, d, 5, 1, K);  // src/ops/linear.cpp:359: returns without work
        double worst = 0;
        for (int p = 0; p < 4; ++p) {
            std::vector<float> Y(Ns[p]);
            ctx.copy_device_to_host(Y.data(), d[p].Y, Y.size() * sizeof(float));
            for (size_t n = 0; n < Ns[p]; ++n) worst = std::fmax(worst, std::fabs(Y[n] - dot_row(X.data(), Ws[p], Ss[p], n, K)));
        }
        report("linear_int4_fused 4 projections", worst <= 1e-4, worst);
    }
    {   // gate / up / SwiGLU, N = 256, K = 512
        const size_t K = 512, N = 256;
        std::vector<float> X(K);
        for (auto& v : X) v = dist(rng);
        auto Wg = fill_w(N * K / 2, 2, 5), Wu = fill_w(N * K / 2, 4, 9);
        auto Sg = fill_s(N * (K / 128)), Su = fill_s(N * (K / 128), 0.020f, 3);
        float* dX = to_device(ctx, X);
        float* dY = static_cast<float*>(ctx.allocate_device(N * sizeof(float)));
        ops::mlp_gate_up_swiglu_int4(ctx.queue(), dY, dX, to_device(ctx, Wg), to_device(ctx, Sg), to_device(ctx, Wu),
                                     to_device(ctx, Su), 1, N, K);
        std::vector<float> Y(N);
        ctx.copy_device_to_host(Y.data(), dY, Y.size() * sizeof(float));
        double worst = 0;
        for (size_t n = 0; n < N; ++n) {
            const double g = dot_row(X.data(), Wg, Sg, n, K), u = dot_row(X.data(), Wu, Su, n, K);
            worst = std::fmax(worst, std::fabs(Y[n] - g / (1.0 + std::exp(-g)) * u));
        }
        report("mlp_gate_up_swiglu_int4", worst <= 1e-4, worst);
    }
    {   // fp16 activations: fp16 out within 5e-3, fp32 out within 1e-4 (tensor-core path)
        const size_t K = 512, N = 256;
        std::vector<half_t> X(K);
        std::vector<float> Xf(K);
        for (size_t i = 0; i < K; ++i) { X[i] = static_cast<half_t>(dist(rng)); Xf[i] = static_cast<float>(X[i]); }
        auto W = fill_w(N * K / 2, 2, 5);
        auto S = fill_s(N * (K / 128));
        half_t* dX = to_device(ctx, X);
        uint8_t* dW = to_device(ctx, W);
        half_t* dS = to_device(ctx, S);
        half_t* dYh = static_cast<half_t*>(ctx.allocate_device(N * sizeof(half_t)));
        float* dYf = static_cast<float*>(ctx.allocate_device(N * sizeof(float)));
        ops::linear_int4(ctx.queue(), dYh, dX, dW, dS, nullptr, 1, N, K);
        ops::linear_int4(ctx.queue(), dYf, dX, dW, dS, nullptr, 1, N, K);
        std::vector<half_t> Yh(N);
        std::vector<float> Yf(N);
        ctx.copy_device_to_host(Yh.data(), dYh, N * sizeof(half_t));
        ctx.copy_device_to_host(Yf.data(), dYf, N * sizeof(float));
        double wh = 0, wf = 0;
        for (size_t n = 0; n < N; ++n) {
            const double e = dot_row(Xf.data(), W, S, n, K);
            wh = std::fmax(wh, std::fabs(static_cast<float>(Yh[n]) - e));
            wf = std::fmax(wf, std::fabs(Yf[n] - e));
        }
        report("linear_int4 f16->f16", wh <= 5e-3, wh);
        report("linear_int4 f16->f32", wf <= 1e-4, wf);
        // invalid shapes are silent no-ops, as in the reference (src/ops/linear.cpp:176)
        ops::linear_int4(ctx.queue(), dYf, dX, dW, dS, nullptr, 0, N, K);
    }
}

void sampling_cases(core::DeviceContext& ctx) {
    {   // argmax over 248320 logits with a planted maximum
        const int64_t V = 248320;
        std::mt19937 rng(48);
        std::uniform_real_distribution<float> dist(-100.0f, 100.0f);
        std::vector<float> L(V);
        for (auto& v : L) v = dist(rng);
        L[123456] = 999.0f;
        float* dL = to_device(ctx, L);
        const int64_t got = ops::argmax(ctx.queue(), dL, V);
        report("argmax 248320", got == 123456, static_cast<double>(got));
        report("argmax_scratch_size", ops::argmax_scratch_size(V) == 970, static_cast<double>(ops::argmax_scratch_size(V)));
        report("argmax null / empty", ops::argmax(ctx.queue(), nullptr, V) == 0 && ops::argmax(ctx.queue(), dL, 0) == 0, 0);
        ctx.free_device(dL);
    }
    {   // acceptance scenarios A-D on vocab 1000, N = 4
        const int64_t V = 1000;
        const size_t N = 4;
        std::vector<float> L(N * V, -10.0f);
        const int64_t peak[4] = {42, 100, 200, 300};
        for (size_t i = 0; i < N; ++i) L[i * V + peak[i]] = 10.0f;
        float* dL = to_device(ctx, L);
        std::vector<int64_t> a = {42, 100, 200, 300};
        auto A = ops::speculative_accept_reject(ctx.queue(), a.data(), N, dL, V);
        report("accept A: all accepted", !A.has_rejected_token && A.num_accepted == 4 && A.accepted_tokens == a &&
                                             A.bonus_or_resampled_token == 300, static_cast<double>(A.num_accepted));
        std::vector<int64_t> b = {42, 100, 999, 300};
        auto B = ops::speculative_accept_reject(ctx.queue(), b.data(), N, dL, V);
        report("accept B: reject at 2", B.has_rejected_token && B.num_accepted == 2 && B.rejected_token == 999 &&
                                            B.bonus_or_resampled_token == 200 && B.num_remaining == 1 && B.num_rejected == 1 &&
                                            B.num_resampled == 1, static_cast<double>(B.num_accepted));
        std::vector<int64_t> c = {999, 100, 200, 300};
        auto C = ops::speculative_accept_reject(ctx.queue(), c.data(), N, dL, V);
        report("accept C: reject at 0", C.has_rejected_token && C.num_accepted == 0 && C.bonus_or_resampled_token == 42 &&
                                            C.num_remaining == 3, static_cast<double>(C.num_accepted));
        std::vector<float> p(N, 1.0f), r(N, 0.1f);
        auto D = ops::speculative_accept_reject(ctx.queue(), a.data(), N, dL, V, p.data(), r.data());
        report("accept D: stochastic, all", !D.has_rejected_token && D.num_accepted == 4, static_cast<double>(D.num_accepted));
        auto E = ops::speculative_accept_reject(ctx.queue(), a.data(), 0, dL, V);
        report("accept: empty input", E.bonus_or_resampled_token == -1 && E.num_accepted == 0, 0);
        ctx.free_device(dL);
    }
}

void arena_cases(std::shared_ptr<core::DeviceContext> ctx) {
    core::DeviceArena arena(ctx, 1 << 20);
    bool ok = arena.capacity() == (1u << 20) && arena.allocate(0) == nullptr;
    void* first = arena.allocate(1000);
    ok = ok && first == arena.base_ptr() && (reinterpret_cast<uintptr_t>(arena.allocate(10)) % 64) == 0;
    for (int step = 0; step < 500; ++step) {   // the same addresses every step: what graph replay relies on
        arena.reset();
        ok = ok && arena.allocate(1000) == first && arena.allocated_bytes() == 1000;
    }
    auto t = arena.allocate_tensor(core::TensorShape{4, 5120}, core::DataType::Float16, 256);
    ok = ok && t.byte_size() == 4 * 5120 * 2 && (reinterpret_cast<uintptr_t>(t.data()) % 256) == 0 && t.shape()[1] == 5120;
    bool threw = false;
    try { arena.allocate(2 << 20); } catch (const std::bad_alloc&) { threw = true; }
    ok = ok && threw;
    void* keep = arena.allocate_persistent(4096);
    arena.reset();
    ok = ok && keep != nullptr && arena.allocated_bytes() == 0 && arena.peak_allocated_bytes() >= 1000;
    threw = false;
    try { arena.persistent_buffer(); } catch (const std::invalid_argument&) { threw = true; }   // first call must size it
    ok = ok && threw && arena.persistent_buffer_capacity() == 0;
    void* pb = arena.persistent_buffer(8192);
    const core::DeviceArena& carena = arena;
    ok = ok && pb && arena.persistent_buffer() == pb && arena.persistent_buffer(100) == pb && carena.persistent_buffer() == pb &&
         arena.persistent_buffer_capacity() == 8192;
    threw = false;
    try { arena.persistent_buffer(8193); } catch (const std::invalid_argument&) { threw = true; }   // refuses to grow
    ok = ok && threw;
    core::DeviceArena moved(std::move(arena));
    ok = ok && moved.capacity() == (1u << 20) && moved.persistent_buffer_capacity() == 8192;
    report("DeviceArena contract", ok, static_cast<double>(moved.peak_allocated_bytes()));
}

}  // namespace

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "--list") == 0) {
        std::puts("linear_int4 linear_int4_fused mlp_gate_up_swiglu_int4 argmax speculative_accept_reject DeviceArena");
        return 0;
    }
    try {
        auto ctx = core::DeviceContext::create(true);
        linear_cases(*ctx);
        sampling_cases(*ctx);
        arena_cases(ctx);
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 2;
    }
    std::printf("%s\n", g_failed ? "SHIM CHECK FAILED" : "shim check passed");
    return g_failed ? 1 : 0;
}
