// A C++ program against the C ABI alone (include/frink_b200.h + libfrink_b200.so, no Python in the process):
// what a maintainer's FFI layer would do.  `abi_check nogpu` exercises the calls that need no device;
// `abi_check gpu` runs Q8_0 matvecs through the host-buffer surface and checks them against a dot product
// computed here.  Exit code 0 = every check passed; each failure prints a line.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "frink_b200.h"

static int failures = 0;
#define CHECK(cond, ...) do { if (!(cond)) { failures++; std::printf("FAIL %s:%d: ", __FILE__, __LINE__); std::printf(__VA_ARGS__); std::printf("\n"); } } while (0)

// IEEE half <-> float, round to nearest even (normal range and zero are all this needs)
static uint16_t f2h(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t m = x & 0x7FFFFFu;
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        m |= 0x800000u;
        const int shift = 14 - e;
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1))) h++;
        return (uint16_t)(sign | h);
    }
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    uint32_t h = ((uint32_t)e << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;
    return (uint16_t)(sign | h);
}
static float h2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FFu;
    uint32_t x;
    if (e == 0) {
        if (m == 0) x = sign;
        else {
            int s = 0;
            uint32_t mm = m;
            while (!(mm & 0x400u)) { mm <<= 1; s++; }
            x = sign | ((uint32_t)(127 - 15 - s + 1) << 23) | ((mm & 0x3FFu) << 13);
        }
    } else x = sign | ((e - 15 + 127) << 23) | (m << 13);
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

// Q8_0 (34 bytes per 32 values: f16 scale, 32 int8), the GGUF layout
static std::vector<uint8_t> encode_q8_0(const std::vector<float>& w, int rows, int cols) {
    std::vector<uint8_t> out((size_t)rows * (cols / 32) * 34);
    for (int r = 0; r < rows; r++)
        for (int b = 0; b < cols / 32; b++) {
            const float* v = &w[(size_t)r * cols + b * 32];
            float amax = 0;
            for (int i = 0; i < 32; i++) amax = std::fmax(amax, std::fabs(v[i]));
            const float d = amax / 127.0f, id = d ? 1.0f / d : 0.0f;
            uint8_t* o = &out[((size_t)r * (cols / 32) + b) * 34];
            const uint16_t dh = f2h(d);
            std::memcpy(o, &dh, 2);
            for (int i = 0; i < 32; i++) o[2 + i] = (uint8_t)(int8_t)std::lround(v[i] * id);
        }
    return out;
}
static std::vector<double> dequant_dot(const std::vector<uint8_t>& q, int rows, int cols, const std::vector<float>& x) {
    std::vector<double> y(rows, 0.0);
    for (int r = 0; r < rows; r++)
        for (int b = 0; b < cols / 32; b++) {
            const uint8_t* o = &q[((size_t)r * (cols / 32) + b) * 34];
            uint16_t dh;
            std::memcpy(&dh, o, 2);
            const double d = h2f(dh);
            for (int i = 0; i < 32; i++) y[r] += d * (int8_t)o[2 + i] * (double)x[b * 32 + i];
        }
    return y;
}
static std::vector<float> randn(size_t n, uint32_t seed, float scale) {
    std::vector<float> v(n);
    uint64_t s = seed * 0x9E3779B97F4A7C15ull + 1;
    for (size_t i = 0; i < n; i++) {
        double acc = 0;
        for (int k = 0; k < 4; k++) { s = s * 6364136223846793005ull + 1442695040888963407ull; acc += (double)(s >> 40) / (double)(1 << 24); }
        v[i] = (float)((acc - 2.0) * 1.7320508) * scale;      // sum of four uniforms: close enough to normal
    }
    return v;
}
static double rel_l2(const float* got, const std::vector<double>& want) {
    double num = 0, den = 0;
    for (size_t i = 0; i < want.size(); i++) { num += (got[i] - want[i]) * (got[i] - want[i]); den += want[i] * want[i]; }
    return std::sqrt(num / (den > 0 ? den : 1));
}

static void no_device_checks() {
    CHECK(fk_block_bytes(FK_Q8_0) == 34 && fk_block_elems(FK_Q8_0) == 32, "Q8_0 block");
    CHECK(fk_block_bytes(FK_Q4_K) == 144 && fk_block_elems(FK_Q4_K) == 256, "Q4_K block");
    CHECK(fk_block_bytes(FK_Q6_K) == 210 && fk_block_elems(FK_Q6_K) == 256, "Q6_K block");
    CHECK(fk_block_bytes(FK_MXFP4) == 17 && fk_block_elems(FK_MXFP4) == 32, "MXFP4 block");
    CHECK(fk_block_bytes(11) < 0, "a kind without kernels has no block size");
    CHECK(fk_init(0, nullptr) == FK_INVALID, "fk_init(null)");
    CHECK(std::strlen(fk_last_error()) > 0, "a failing call leaves a message");
    CHECK(fk_device_info(nullptr, nullptr, 0, nullptr, nullptr) == FK_INVALID, "device_info(null)");
    CHECK(fk_launch_matvec(nullptr, FK_Q8_0, nullptr, 0, nullptr, 1, 34, 1, nullptr) != FK_OK, "launch_matvec(null)");
    CHECK(fk_launch_matvec_multi(nullptr, nullptr, 32, nullptr, 1, nullptr) == FK_INVALID, "launch_matvec_multi(null)");
    CHECK(fk_comm_channel_bytes(2, 1024) == (size_t)(2 * 2 * 1024 * 8 + 1024 * 4), "channel bytes");
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "nogpu";
    no_device_checks();
    fk_ctx* ctx = nullptr;
    const int rc = fk_init(0, &ctx);
    if (mode == "nogpu") {
        // with no device this must be a clean refusal, never a crash and never a context
        if (rc != FK_OK) {
            CHECK(rc == FK_DRIVER_INIT || rc == FK_UNSUPPORTED, "fk_init without a device returned %d", rc);
            CHECK(ctx == nullptr && std::strlen(fk_last_error()) > 0, "no context, a message");
        } else fk_destroy(ctx);
        std::printf("%s\n", failures ? "abi_check: FAILED" : "abi_check: ok (no device needed)");
        return failures ? 1 : 0;
    }
    CHECK(rc == FK_OK, "fk_init: %s", fk_last_error());
    if (rc != FK_OK) return 1;
    char name[128];
    int sms = 0;
    size_t mem = 0;
    CHECK(fk_device_info(ctx, name, sizeof name, &sms, &mem) == FK_OK && sms > 0 && mem > 0, "device_info");

    const int cols = 1024, ffn = 512, rows = 384;
    const std::vector<float> x = randn(cols, 1, 1.0f);
    const std::vector<uint8_t> wq = encode_q8_0(randn((size_t)rows * cols, 2, 0.05f), rows, cols);
    const std::vector<uint8_t> wk = encode_q8_0(randn((size_t)ffn * cols, 3, 0.05f), ffn, cols);
    const std::vector<uint8_t> wu = encode_q8_0(randn((size_t)ffn * cols, 4, 0.05f), ffn, cols);
    const std::vector<uint8_t> wd = encode_q8_0(randn((size_t)rows * ffn, 5, 0.05f), rows, ffn);
    const int rbc = cols / 32 * 34, rbf = ffn / 32 * 34;

    // one matvec; the activation is quantized to 8 bits on the device, so the distance to the dot with the raw x is ~5e-3
    std::vector<float> y(rows, NAN);
    CHECK(fk_launch_matvec(ctx, FK_Q8_0, wq.data(), wq.size(), x.data(), rows, rbc, cols / 32, y.data()) == FK_OK, "launch_matvec: %s", fk_last_error());
    const double e1 = rel_l2(y.data(), dequant_dot(wq, rows, cols, x));
    CHECK(e1 < 1.5e-2, "launch_matvec rel l2 %g", e1);

    // the same twice gives the same bits, and a second call finds the weights resident (no second upload)
    uint64_t h2d0 = 0, h2d1 = 0;
    fk_counters(ctx, &h2d0, nullptr, nullptr, 0);
    std::vector<float> y2(rows, NAN);
    CHECK(fk_launch_matvec(ctx, FK_Q8_0, wq.data(), wq.size(), x.data(), rows, rbc, cols / 32, y2.data()) == FK_OK, "launch_matvec again");
    fk_counters(ctx, &h2d1, nullptr, nullptr, 0);
    CHECK(std::memcmp(y.data(), y2.data(), rows * 4) == 0, "run-to-run bits");
    CHECK(h2d1 - h2d0 == (uint64_t)cols * 4, "second call uploaded %llu bytes, x is %d", (unsigned long long)(h2d1 - h2d0), cols * 4);

    // launch_matvec_multi = the single launches
    fk_matvec_launch ls[2] = {{FK_Q8_0, wq.data(), wq.size(), rows, rbc, cols / 32}, {FK_Q8_0, wk.data(), wk.size(), ffn, rbc, cols / 32}};
    std::vector<float> m0(rows, NAN), m1(ffn, NAN), s1(ffn, NAN);
    float* outs[2] = {m0.data(), m1.data()};
    CHECK(fk_launch_matvec_multi(ctx, x.data(), cols, ls, 2, outs) == FK_OK, "launch_matvec_multi: %s", fk_last_error());
    CHECK(fk_launch_matvec(ctx, FK_Q8_0, wk.data(), wk.size(), x.data(), ffn, rbc, cols / 32, s1.data()) == FK_OK, "launch_matvec (k)");
    CHECK(std::memcmp(m0.data(), y.data(), rows * 4) == 0 && std::memcmp(m1.data(), s1.data(), ffn * 4) == 0, "multi equals the single launches");

    // launch_dense_ffn_swiglu against gate / up / SiLU / down composed here from the device's own gate and up
    fk_matvec_launch lg = {FK_Q8_0, wk.data(), wk.size(), ffn, rbc, cols / 32}, lu = {FK_Q8_0, wu.data(), wu.size(), ffn, rbc, cols / 32};
    fk_matvec_launch ld = {FK_Q8_0, wd.data(), wd.size(), rows, rbf, ffn / 32};
    std::vector<float> f(rows, NAN), up(ffn, NAN), act(ffn);
    CHECK(fk_launch_dense_ffn_swiglu(ctx, &lg, &lu, &ld, x.data(), cols, f.data()) == FK_OK, "launch_dense_ffn_swiglu: %s", fk_last_error());
    CHECK(fk_launch_matvec(ctx, FK_Q8_0, wu.data(), wu.size(), x.data(), ffn, rbc, cols / 32, up.data()) == FK_OK, "launch_matvec (up)");
    for (int i = 0; i < ffn; i++) act[i] = s1[i] / (1.0f + std::exp(-s1[i])) * up[i];
    const double e2 = rel_l2(f.data(), dequant_dot(wd, rows, ffn, act));
    CHECK(e2 < 1.5e-2, "dense ffn rel l2 %g", e2);

    // refusals: a row size that does not match, a kind without kernels (UNSUPPORTED keeps its meaning: use another path)
    CHECK(fk_launch_matvec(ctx, FK_Q8_0, wq.data(), wq.size(), x.data(), rows, rbc + 2, cols / 32, y.data()) == FK_INVALID, "bad row_bytes");
    CHECK(fk_launch_matvec(ctx, 11, wq.data(), wq.size(), x.data(), rows, rbc, cols / 32, y.data()) == FK_UNSUPPORTED, "kind 11");
    int code = -1;
    CHECK(fk_device_error(ctx, &code, 1) == FK_OK && code == 0, "device error word %d", code);
    fk_forget_resident(ctx);
    fk_destroy(ctx);
    std::printf("%s (%s, %d SMs; matvec %.2e, ffn %.2e)\n", failures ? "abi_check: FAILED" : "abi_check: ok", name, sms, e1, e2);
    return failures ? 1 : 0;
}
