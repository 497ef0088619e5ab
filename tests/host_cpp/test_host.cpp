// test_host.cpp — exercises the C++ host layer (goml_b200/host/goml_cuda.hpp) the way goml's Go tests exercise
// backend/cuda: library search rules, error text, dispatcher table (no GPU), and on a GPU the closed-form LSE
// tests of backend/cuda/fa_forward_test.go:112-288, the GEMM self-check of libs/fp8_gemm_bench.cu:81-141, a
// quantise -> attention chain with device-resident scales against a CPU double loop
// (backend/cuda/fa_chain_cpuref_test.go:268: floor 5e-3), and head sharding through the device manager.
//   usage: test_host cpu <libs_dir>   |   test_host gpu
#include <cstring>
#include <iostream>
#include <vector>

#include "../../goml_b200/host/goml_cuda.hpp"

using namespace goml::cuda;

static int fails = 0;
#define CHECK(cond) do { if (!(cond)) { std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); fails++; } } while (0)

static float e4m3_decode(uint8_t v) {
    int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
    float r = e == 0 ? std::ldexp((float)m, -9) : std::ldexp(1.0f + m / 8.0f, e - 7);
    return s ? -r : r;
}
static uint8_t e4m3_encode_exact(float f) {  // for values that are exactly representable
    for (int c = 0; c < 256; c++)
        if ((c & 0x7f) != 0x7f && e4m3_decode((uint8_t)c) == f && !(c == 0x80)) return (uint8_t)c;
    return 0x7f;
}

template <class F>
static std::string thrown(F f) {
    try { f(); } catch (const Error& e) { return e.what(); }
    return "";
}

static int run_cpu(const char* libs_dir) {
    // library search (arch.go:57-101)
    setenv("GOML_LIBS_DIR", libs_dir, 1);
    CHECK(LibsDir() == libs_dir);
    CHECK(resolveLib("libfp8gemm.so") == std::string(libs_dir) + "/libfp8gemm.so");
    CHECK(resolveLib("libnothing_here.so") == "libnothing_here.so");
    // error text (fp8_gemm.go:57-61): CUDA error code in the message
    CHECK(thrown([] { FP8GEMM(8, 8, 24, 16, 16, 16, ModeSinglesync, 0); }) == "fp8_gemm: CUDA error 1");
    CHECK(thrown([] { FP8GEMMScaled(8, 8, 32, 16, 16, 16, 1.0f, 0, 0, 9, 0); }) == "fp8_gemm_scaled: CUDA error 1");
    CHECK(thrown([] { FP8GEMMAccumulateF32(8, 8, 32, 16, 16, 0, 1.0f, 0, 0, 0); }) == "fp8_gemm_accumulate_f32: CUDA error 1");
    // status strings and dispatcher (fa_forward.go:36-60; libs/fa_sm120/go/gofa/gofa_test.go:15-37)
    FALoad();
    CHECK(FAStatusString(FA_OK) == "OK");
    CHECK(FAStatusString(FA_ERR_INVALID_ARG) == "invalid argument");
    CHECK(FAVersion().find("sm100a") != std::string::npos);
    struct { int bh, sl, hd, ca, w, want; } rows[] = {
        {64, 8192, 128, 0, 0, 100}, {128, 8192, 128, 0, 0, 100}, {4, 1024, 128, 0, 0, 103}, {4, 4096, 128, 0, 0, 102},
        {16, 4096, 128, 0, 0, 105}, {4, 8192, 128, 1, 1024, 104}, {64, 8192, 128, 1, 1024, 101}, {64, 8192, 64, 0, 0, 200},
        {4, 1024, 64, 0, 0, 201}, {64, 8192, 96, 0, 0, -1}};
    for (auto& r : rows) CHECK(FADispatchSelect(r.bh, r.sl, r.hd, r.ca, r.w) == r.want);
    // partitions
    for (long long total : {1LL, 7LL, 128LL, 129LL})
        for (int ws : {1, 2, 3, 8}) {
            long long at = 0;
            for (int r = 0; r < ws; r++) { Shard s = ShardHeads(total, ws, r); CHECK(s.begin == at); at = s.end; }
            CHECK(at == total);
        }
    CHECK(ShardRows(16384, 8, 3).begin == 6144 && ShardRows(16384, 8, 3).end == 8192);
    CHECK(ShardRows(300, 2, 1).begin == 256 && ShardRows(300, 2, 1).end == 300);
    // block glue: argument errors before any launch, same message shape
    CHECK(thrown([] { SwiGLUQuantize(64, 64, 64, 64, 2, 40, 0); }) == "fp8_swiglu_quantize: CUDA error 1");
    CHECK(thrown([] { ResidualAdd(64, 64, 12, 0); }) == "fp8_residual_add: CUDA error 1");
    CHECK(thrown([] { FP8GEMMSwiGLU(8, 0, 32, 16, 16, 16, 1.0f, 0, 0, 16, 0); }) == "fp8_gemm_swiglu: CUDA error 1");
    CHECK(thrown([] { FP8GEMMFP8Out(8, 8, 32, 16, 16, 0, 1.0f, 0, 0, 0, 0, 0); }) == "fp8_gemm_fp8out: CUDA error 1");
    CHECK(thrown([] { fp8_decode_append_args_t a{}; a.batch = 1; DecodeRopeAppend(a); }) == "fp8_decode_rope_append: CUDA error 1");
    {   // weight layout for the SwiGLU GEMM: F = 70 -> three blocks of 32 columns, the last one mostly padding
        const int F = 70, K = 4;
        std::vector<uint8_t> w((size_t)2 * F * K);
        for (size_t i = 0; i < w.size(); i++) w[i] = (uint8_t)(i / K + 1);   // row index + 1 in every byte of a row
        const auto wi = InterleaveGateUp(w, F, K);
        CHECK(wi.size() == (size_t)2 * 96 * K);
        // rows 0..31 gate 0..31, rows 32..63 up 0..31, rows 64..95 gate 32..63, ..., rows 128..133 gate 64..69, then zeros
        CHECK(wi[0] == 1 && wi[(size_t)31 * K] == 32 && wi[(size_t)32 * K] == (uint8_t)(F + 1) && wi[(size_t)64 * K] == 33 &&
              wi[(size_t)128 * K] == 65 && wi[(size_t)133 * K] == 70 && wi[(size_t)134 * K] == 0 &&
              wi[(size_t)160 * K] == (uint8_t)(F + 65) && wi[(size_t)166 * K] == 0);
    }
    return fails;
}

template <class T>
struct DevBuf {
    T* p = nullptr;
    size_t n;
    explicit DevBuf(size_t n_) : n(n_) { cudaMalloc(&p, n * sizeof(T)); cudaMemset(p, 0, n * sizeof(T)); }
    ~DevBuf() { cudaFree(p); }
    uintptr_t addr() const { return reinterpret_cast<uintptr_t>(p); }
    void up(const std::vector<T>& h) { cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice); }
    std::vector<T> down() const { std::vector<T> h(n); cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost); return h; }
};
static float half_to_float(uint16_t h) {
    int s = h >> 15, e = (h >> 10) & 31, m = h & 1023;
    float r = e == 0 ? std::ldexp((float)m, -24) : (e == 31 ? INFINITY : std::ldexp(1.0f + m / 1024.0f, e - 15));
    return s ? -r : r;
}

static int run_gpu() {
    std::printf("version %s\n", FAVersion().c_str());
    DeviceManager mgr;
    auto& dev = mgr.Use(0);
    FAContext& ctx = *dev.fa;
    const uintptr_t stream = reinterpret_cast<uintptr_t>(dev.stream);

    {   // TestFAForwardTrain_L_Uniform / _L_Layout (fa_forward_test.go:112-288)
        const int bh = 3, sl = 280, hd = 128;
        const size_t n = (size_t)bh * sl * hd;
        std::vector<uint8_t> ones(n, 0x38), qh(n);
        const uint8_t code[3] = {0x38, 0x40, 0x48};  // 1, 2, 4 per head
        for (int h = 0; h < bh; h++) std::fill(qh.begin() + (size_t)h * sl * hd, qh.begin() + (size_t)(h + 1) * sl * hd, code[h]);
        DevBuf<uint8_t> q(n), k(n), v(n);
        DevBuf<uint16_t> o(n);
        DevBuf<float> l((size_t)bh * sl);
        k.up(ones); v.up(ones);
        for (int variant = 0; variant < 2; variant++) {
            q.up(variant == 0 ? ones : qh);
            ctx.ForwardTrain(q.addr(), k.addr(), v.addr(), o.addr(), l.addr(), bh, sl, hd, 0, 0, 1.0f / std::sqrt((float)hd), stream);
            cudaStreamSynchronize(dev.stream);
            auto L = l.down();
            for (int h = 0; h < bh; h++) {
                const double want = (variant == 0 ? 1.0 : std::ldexp(1.0, h)) * std::sqrt((double)hd) + std::log((double)sl);
                double worst = 0;
                for (int i = 0; i < sl; i++) worst = std::max(worst, std::fabs(L[(size_t)h * sl + i] - want) / want);
                CHECK(worst <= 5e-3);
            }
            if (variant == 0) {
                auto O = o.down();
                double worst = 0;
                for (size_t i = 0; i < n; i++) worst = std::max(worst, (double)std::fabs(half_to_float(O[i]) - 1.0f));
                CHECK(worst <= 1e-3);
            }
        }
    }
    {   // GEMM self-check (libs/fp8_gemm_bench.cu:81-141): srand(42), ((rand()%16)-8)*0.25, gate max(1, 0.05|ref|)
        const int M = 128, N = 128, K = 128;
        std::vector<uint8_t> hA((size_t)M * K), hB((size_t)N * K);
        srand(42);
        for (auto& x : hA) x = e4m3_encode_exact(((float)(rand() % 16) - 8.0f) * 0.25f);
        for (auto& x : hB) x = e4m3_encode_exact(((float)(rand() % 16) - 8.0f) * 0.25f);
        DevBuf<uint8_t> A(hA.size()), B(hB.size());
        DevBuf<uint16_t> C((size_t)M * N);
        A.up(hA); B.up(hB);
        for (int mode : {ModeOriginal, ModeSinglesync}) {
            FP8GEMM(M, N, K, A.addr(), B.addr(), C.addr(), mode, stream);
            cudaStreamSynchronize(dev.stream);
            auto hC = C.down();
            int bad = 0;
            for (int m = 0; m < M; m++)
                for (int nn = 0; nn < N; nn++) {
                    float sum = 0;
                    for (int kk = 0; kk < K; kk++) sum += e4m3_decode(hA[m * K + kk]) * e4m3_decode(hB[nn * K + kk]);
                    if (std::fabs(half_to_float(hC[m * N + nn]) - sum) > std::fmax(1.0f, 0.05f * std::fabs(sum))) bad++;
                }
            CHECK(bad == 0);
        }
        CHECK(FP8GEMMDeviceStatus() == 0);
    }
    {   // quantise (unit convention) -> attention with device-resident scales; vs a CPU double loop, floor 5e-3
        const int bh = 2, sl = 128, hd = 128;
        const size_t n = (size_t)bh * sl * hd;
        std::vector<float> x[3];
        srand(7);
        for (auto& t : x) { t.resize(n); for (auto& e : t) e = (float)rand() / RAND_MAX * 2.0f - 1.0f; }
        DevBuf<float> xf(n), sc(6);
        DevBuf<uint8_t> q(n), k(n), v(n);
        DevBuf<uint8_t>* codes[3] = {&q, &k, &v};
        for (int t = 0; t < 3; t++) {
            xf.up(x[t]);
            QuantizeF32ToF8E4M3Unit(xf.addr(), codes[t]->addr(), sc.addr() + 8 * t, sc.addr() + 8 * t + 4, n, stream);
            cudaStreamSynchronize(dev.stream);
        }
        DevBuf<uint16_t> o(n);
        DevBuf<float> l((size_t)bh * sl);
        fa_forward_args_t a{};
        a.q = q.p; a.k = k.p; a.v = v.p; a.o = o.p; a.l_out = l.p;
        a.batch_heads = bh; a.seq_len = sl; a.head_dim = hd; a.causal = 1; a.window = 0;
        a.scale = 1.0f / std::sqrt((float)hd); a.v_descale = 1.0f;
        a.scale_q_dev = sc.p; a.scale_k_dev = sc.p + 2; a.scale_v_dev = sc.p + 4;
        a.stream = reinterpret_cast<fa_stream_t>(dev.stream);
        ctx.ForwardEx(a);
        cudaStreamSynchronize(dev.stream);
        ctx.DeviceStatus();
        auto hq = q.down(), hk = k.down(), hv = v.down();
        auto hs = sc.down();
        auto hO = o.down();
        auto hL = l.down();
        const double scale = (double)a.scale * hs[0] * hs[2];
        double worstO = 0, worstL = 0;
        std::vector<double> p(sl);
        for (int h = 0; h < bh; h++)
            for (int i = 0; i < sl; i++) {
                double mx = -INFINITY;
                for (int j = 0; j <= i; j++) {
                    double s = 0;
                    for (int d = 0; d < hd; d++) s += (double)e4m3_decode(hq[((size_t)h * sl + i) * hd + d]) * e4m3_decode(hk[((size_t)h * sl + j) * hd + d]);
                    p[j] = s * scale;
                    mx = std::max(mx, p[j]);
                }
                double sum = 0;
                for (int j = 0; j <= i; j++) { p[j] = std::exp(p[j] - mx); sum += p[j]; }
                worstL = std::max(worstL, std::fabs(hL[(size_t)h * sl + i] - (mx + std::log(sum))));
                for (int d = 0; d < hd; d++) {
                    double acc = 0;
                    for (int j = 0; j <= i; j++) acc += p[j] * e4m3_decode(hv[((size_t)h * sl + j) * hd + d]);
                    worstO = std::max(worstO, std::fabs(half_to_float(hO[((size_t)h * sl + i) * hd + d]) - acc / sum * hs[4]));
                }
            }
        std::printf("chain: worst |O-ref| %.3e  worst |L-ref| %.3e\n", worstO, worstL);
        CHECK(worstO <= 5e-3 && worstL <= 5e-3);

        // head sharding through the manager: every shard computed on its own device (round-robin over the
        // devices present) gives the bytes of the unsharded call
        const int world = 2;
        std::vector<uint16_t> sharded(n);
        for (int r = 0; r < world; r++) {
            const Shard s = ShardHeads(bh, world, r);
            auto& d = mgr.Use(r % mgr.Count());
            const size_t off = (size_t)s.begin * sl * hd, cnt = (size_t)(s.end - s.begin) * sl * hd;
            DevBuf<uint8_t> sq(cnt), sk(cnt), sv(cnt);
            DevBuf<uint16_t> so(cnt);
            DevBuf<float> ssc(6);
            sq.up(std::vector<uint8_t>(hq.begin() + off, hq.begin() + off + cnt));
            sk.up(std::vector<uint8_t>(hk.begin() + off, hk.begin() + off + cnt));
            sv.up(std::vector<uint8_t>(hv.begin() + off, hv.begin() + off + cnt));
            ssc.up(hs);
            fa_forward_args_t b = a;
            b.q = sq.p; b.k = sk.p; b.v = sv.p; b.o = so.p; b.l_out = nullptr;
            b.batch_heads = (int)(s.end - s.begin);
            b.scale_q_dev = ssc.p; b.scale_k_dev = ssc.p + 2; b.scale_v_dev = ssc.p + 4;
            b.stream = reinterpret_cast<fa_stream_t>(d.stream);
            d.fa->ForwardEx(b);
            cudaStreamSynchronize(d.stream);
            auto part = so.down();
            std::copy(part.begin(), part.end(), sharded.begin() + off);
        }
        CHECK(sharded == hO);
    }
    {   // block glue through the host layer: residual add exact, SwiGLU codes decode to silu(g)*u within one e4m3 step
        const int rows = 8, F = 64;
        std::vector<float> xs(rows * F);
        std::vector<uint16_t> yb(rows * F), gu(rows * 2 * F);
        auto bf16 = [](float f) { uint32_t u; std::memcpy(&u, &f, 4); return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1)) >> 16); };
        auto bf2f = [](uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; std::memcpy(&f, &u, 4); return f; };
        for (int i = 0; i < rows * F; i++) { xs[i] = std::sin(0.37f * i); yb[i] = bf16(std::cos(0.11f * i)); }
        for (int i = 0; i < rows * 2 * F; i++) gu[i] = bf16(3.0f * std::sin(0.05f * i + 1.0f));
        DevBuf<float> dx(rows * F), sa(2);
        DevBuf<uint16_t> dy(rows * F), dgu(rows * 2 * F);
        DevBuf<uint8_t> dq(rows * F);
        dx.up(xs); dy.up(yb); dgu.up(gu);
        ResidualAdd(dx.addr(), dy.addr(), (size_t)rows * F, 0);
        SwiGLUQuantize(dgu.addr(), dq.addr(), sa.addr(), sa.addr() + 4, rows, F, 0);
        cudaDeviceSynchronize();
        auto hx = dx.down();
        auto hq = dq.down();
        auto hs = sa.down();
        bool exact = true;
        double worst = 0, amax = 0;
        for (int i = 0; i < rows * F; i++) exact = exact && hx[i] == xs[i] + bf2f(yb[i]);
        for (int r = 0; r < rows; r++)
            for (int c = 0; c < F; c++) {
                const double g = bf2f(gu[r * 2 * F + c]), u = bf2f(gu[r * 2 * F + F + c]);
                const double ref = g / (1.0 + std::exp(-g)) * u;
                amax = std::max(amax, std::fabs(ref));
                worst = std::max(worst, std::fabs(e4m3_decode(hq[r * F + c]) * hs[0] - ref) / std::max(std::fabs(ref), 1e-3));
            }
        std::printf("glue: residual add exact %d, swiglu worst relative step %.3f, amax %.6f vs %.6f\n", (int)exact, worst, hs[1], amax);
        CHECK(exact && worst <= 0.07 && std::fabs(hs[1] - amax) <= 1e-5 * amax && std::fabs(hs[0] - hs[1] / 448.0f) <= 1e-7f);
    }
    // argument errors carry the reference's message shape (fa_forward.go:176-181)
    const std::string msg = thrown([&] { ctx.ForwardTrain(0, 16, 16, 16, 0, 1, 64, 128, 0, 0, 1.0f, 0); });
    CHECK(msg.rfind("fa_forward_train: invalid argument (", 0) == 0);
    return fails;
}

// "block <dir> B S d H F": the FP8 decoder block through goml::cuda::nn, fed from files written by the Python test
// (x, weights and norm gains as raw fp32); writes the updated residual stream to <dir>/y.f32.
static std::vector<float> read_f32(const std::string& path, size_t n) {
    std::vector<float> v(n);
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f || std::fread(v.data(), 4, n, f) != n) throw std::runtime_error("cannot read " + path);
    std::fclose(f);
    return v;
}
static int run_block(const std::string& dir, int B, int S, int d, int H, int F) {
    namespace N = goml::cuda::nn;
    const int T = B * S, hd = d / H, Fp = (F + 31) / 32 * 32;
    auto fa = FAContext::FACreate();
    // weights: upload fp32, quantise on the device with the library's quantiser (scale = amax/448)
    struct W { DevBuf<float> f; DevBuf<uint8_t> q; DevBuf<float> sa; W(size_t n) : f(n), q(n), sa(2) {} };
    auto load = [&](const char* name, size_t n) {
        auto w = std::unique_ptr<W>(new W(n));
        w->f.up(read_f32(dir + "/" + name, n));
        QuantizeF32ToF8E4M3(w->f.addr(), w->q.addr(), w->sa.addr(), w->sa.addr() + 4, n, 0);
        return w;
    };
    auto wqkv = load("wqkv.f32", (size_t)3 * d * d), wo = load("wo.f32", (size_t)d * d);
    auto wgu = load("wgate_up.f32", (size_t)2 * F * d), wdn = load("wdown.f32", (size_t)d * F);
    cudaDeviceSynchronize();
    DevBuf<uint8_t> wgui((size_t)2 * Fp * d);
    wgui.up(InterleaveGateUp(wgu->q.down(), F, d));
    DevBuf<float> g1(d), g2(d), h((size_t)T * d);
    g1.up(read_f32(dir + "/g1.f32", d)); g2.up(read_f32(dir + "/g2.f32", d)); h.up(read_f32(dir + "/x.f32", (size_t)T * d));
    // work buffers
    DevBuf<float> rstd(T), sx(2), so(2), sh(2), s3(6), cosb((size_t)S * hd / 2), sinb((size_t)S * hd / 2);
    DevBuf<uint8_t> xq((size_t)T * d), oq((size_t)T * d), hq((size_t)T * F), qc((size_t)T * d), kc((size_t)T * d), vc((size_t)T * d);
    DevBuf<uint16_t> qkv((size_t)T * 3 * d), o16((size_t)T * d), hb((size_t)T * F);
    RopeTable(cosb.addr(), sinb.addr(), S, hd, 10000.0f, 0);
    N::FP8DecoderBlock blk;
    blk.d = d; blk.H = H; blk.F = F; blk.eps = 1e-5f; blk.fa = fa.get();
    blk.qkv = {d, 3 * d, {wqkv->q.addr(), wqkv->sa.addr(), wqkv->sa.addr() + 4}};
    blk.o = {d, d, {wo->q.addr(), wo->sa.addr(), wo->sa.addr() + 4}};
    blk.down = {F, d, {wdn->q.addr(), wdn->sa.addr(), wdn->sa.addr() + 4}};
    blk.gate_up_interleaved = {wgui.addr(), wgu->sa.addr(), wgu->sa.addr() + 4};
    blk.norm1 = g1.addr(); blk.norm2 = g2.addr();
    N::BlockBuffers w;
    w.rstd = rstd.addr();
    w.xq = {xq.addr(), sx.addr(), sx.addr() + 4}; w.oq = {oq.addr(), so.addr(), so.addr() + 4}; w.hq = {hq.addr(), sh.addr(), sh.addr() + 4};
    w.qkv = qkv.addr(); w.qc = qc.addr(); w.kc = kc.addr(); w.vc = vc.addr();
    w.qkv_scales = s3.addr(); w.qkv_amax = s3.addr() + 12; w.o = o16.addr(); w.hb = hb.addr(); w.cos = cosb.addr(); w.sin = sinb.addr();
    blk.Forward(h.addr(), B, S, w, 0);
    cudaDeviceSynchronize();
    fa->DeviceStatus();
    CHECK(FP8GEMMDeviceStatus() == 0);
    auto y = h.down();
    FILE* f = std::fopen((dir + "/y.f32").c_str(), "wb");
    if (!f || std::fwrite(y.data(), 4, y.size(), f) != y.size()) throw std::runtime_error("cannot write y.f32");
    std::fclose(f);
    return fails;
}

int main(int argc, char** argv) {
    try {
        if (argc >= 8 && !std::strcmp(argv[1], "block")) {
            int f = run_block(argv[2], std::atoi(argv[3]), std::atoi(argv[4]), std::atoi(argv[5]), std::atoi(argv[6]), std::atoi(argv[7]));
            std::printf("%s\n", f ? "FAILED" : "block ok");
            return f != 0;
        }
        if (argc >= 3 && !std::strcmp(argv[1], "cpu")) { int f = run_cpu(argv[2]); std::printf("%s\n", f ? "FAILED" : "cpu ok"); return f != 0; }
        if (argc >= 2 && !std::strcmp(argv[1], "gpu")) { int f = run_gpu(); std::printf("%s\n", f ? "FAILED" : "gpu ok"); return f != 0; }
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 2;
    }
    std::printf("usage: test_host cpu <libs_dir> | gpu\n");
    return 64;
}
