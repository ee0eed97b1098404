// pin_formats.cu -- host-only check of the oracle's number formats against CUDA's own host
// conversions.  TEST INFRASTRUCTURE ONLY; needs nvcc but no GPU.  Exit code 0 = every value agrees.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>

extern "C" {
float blzo_f16_to_f32(uint16_t);
uint16_t blzo_f32_to_f16(float);
float blzo_bf16_to_f32(uint16_t);
uint16_t blzo_f32_to_bf16(float);
float blzo_e4m3_to_f32(uint8_t);
uint8_t blzo_f32_to_e4m3(float);
float blzo_e2m1_to_f32(uint8_t);
uint8_t blzo_f32_to_e2m1(float);
}

static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static bool same(float a, float b) { return (std::isnan(a) && std::isnan(b)) || f2u(a) == f2u(b); }

static uint32_t lcg(uint32_t& s) { s = s * 1664525u + 1013904223u; return s; }

int main() {
    long bad = 0, checked = 0;

    // decode tables
    for (uint32_t h = 0; h < 65536; h++) {
        __half_raw r; r.x = (uint16_t)h;
        float want = __half2float(__half(r));
        if (!same(want, blzo_f16_to_f32((uint16_t)h))) { if (bad++ < 5) printf("f16 decode %04x\n", h); }
        __nv_bfloat16_raw br; br.x = (uint16_t)h;
        float wantb = __bfloat162float(__nv_bfloat16(br));
        if (!same(wantb, blzo_bf16_to_f32((uint16_t)h))) { if (bad++ < 5) printf("bf16 decode %04x\n", h); }
        checked += 2;
    }
    for (uint32_t b = 0; b < 256; b++) {
        __half_raw r = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
        float want = __half2float(__half(r));
        if (!same(want, blzo_e4m3_to_f32((uint8_t)b))) { if (bad++ < 5) printf("e4m3 decode %02x\n", b); }
        checked++;
    }
    for (uint32_t n = 0; n < 16; n++) {
        __half_raw r = __nv_cvt_fp4_to_halfraw((__nv_fp4_storage_t)n, __NV_E2M1);
        float want = __half2float(__half(r));
        if (!same(want, blzo_e2m1_to_f32((uint8_t)n))) { if (bad++ < 5) printf("e2m1 decode %x\n", n); }
        checked++;
    }

    // encoders: every fp16 value, every midpoint between neighbouring codes, and random fp32 patterns
    auto check_enc = [&](float x) {
        if (!std::isnan(x)) {
            uint16_t hw = __half_raw(__float2half_rn(x)).x;
            if (hw != blzo_f32_to_f16(x)) { if (bad++ < 5) printf("f16 encode %08x want %04x got %04x\n", f2u(x), hw, blzo_f32_to_f16(x)); }
            uint16_t bw = __nv_bfloat16_raw(__float2bfloat16_rn(x)).x;
            if (bw != blzo_f32_to_bf16(x)) { if (bad++ < 5) printf("bf16 encode %08x want %04x got %04x\n", f2u(x), bw, blzo_f32_to_bf16(x)); }
            checked += 2;
        }
        uint8_t e8 = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
        uint8_t o8 = blzo_f32_to_e4m3(x);
        bool nan8 = std::isnan(x);
        if (nan8 ? ((e8 & 0x7f) != (o8 & 0x7f)) : (e8 != o8)) { if (bad++ < 5) printf("e4m3 encode %08x (%g) want %02x got %02x\n", f2u(x), x, e8, o8); }
        if (!std::isnan(x)) {
            uint8_t e4 = (uint8_t)__nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest) & 15;
            uint8_t o4 = blzo_f32_to_e2m1(x);
            if (e4 != o4) { if (bad++ < 5) printf("e2m1 encode %08x (%g) want %x got %x\n", f2u(x), x, e4, o4); }
            checked++;
        }
        checked++;
    };
    for (uint32_t h = 0; h < 65536; h++) {
        float x = blzo_f16_to_f32((uint16_t)h);
        check_enc(x);
        if (!std::isnan(x) && !std::isinf(x)) {
            check_enc(u2f(f2u(x) + 1));
            if (f2u(x) & 0x7fffffffu) check_enc(u2f(f2u(x) - 1));
        }
    }
    // exact midpoints of E4M3 and E2M1 neighbours and their fp32 neighbours
    for (uint32_t b = 0; b < 0x7e; b++) {
        float m = 0.5f * (blzo_e4m3_to_f32((uint8_t)b) + blzo_e4m3_to_f32((uint8_t)(b + 1)));
        for (int s = 0; s < 2; s++) {
            float v = s ? -m : m;
            check_enc(v); check_enc(u2f(f2u(v) + 1)); check_enc(u2f(f2u(v) - 1));
        }
    }
    for (uint32_t n = 0; n < 7; n++) {
        float m = 0.5f * (blzo_e2m1_to_f32((uint8_t)n) + blzo_e2m1_to_f32((uint8_t)(n + 1)));
        for (int s = 0; s < 2; s++) {
            float v = s ? -m : m;
            check_enc(v); check_enc(u2f(f2u(v) + 1)); check_enc(u2f(f2u(v) - 1));
        }
    }
    uint32_t seed = 12345u;
    for (int i = 0; i < 4000000; i++) {
        uint32_t u = lcg(seed) ^ (lcg(seed) >> 11);
        check_enc(u2f(u));
        // values concentrated in the E4M3 / E2M1 range
        float y = ((float)(lcg(seed) >> 8) / 16777216.0f - 0.5f) * 1000.0f;
        check_enc(y);
        check_enc(y * 0.01f);
    }
    float specials[] = {0.0f, -0.0f, INFINITY, -INFINITY, NAN, 448.0f, 464.0f, 465.0f, 480.0f, 1e9f, 6.0f, 7.0f, 65504.0f, 65519.9f, 65520.0f};
    for (float v : specials) check_enc(v);

    printf("pin_formats: checked %ld conversions, %ld mismatches\n", checked, bad);
    return bad ? 1 : 0;
}
