// Known-answer generator built against the REFERENCE's own cccc/types.h (found through the
// include path given by the Makefile; nothing of the reference is copied here).
// Test infrastructure only.  It prints, as text, what the reference's host codecs produce:
//   e5m2_decode / e4m3_decode : float bits of all 256 byte values
//   fp4_table                 : float bits of the 16 nibble values
//   e5m2_encode / e4m3_encode / fp4_encode : byte produced for each probe float
//   bf16_host                 : the (truncating) host bfloat16(float) constructor
// Probe floats are read as hex bit patterns from stdin, one per line.
#include "types.h"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

static uint32_t bits(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
static float fromBits(uint32_t u)
{
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

int main()
{
    std::printf("e5m2_decode");
    for (int b = 0; b < 256; b++)
    {
        cccc::fp8_e5m2 v;
        v.bits = (uint8_t)b;
        std::printf(" %08x", bits((float)v));
    }
    std::printf("\ne4m3_decode");
    for (int b = 0; b < 256; b++)
    {
        cccc::fp8_e4m3 v;
        v.bits = (uint8_t)b;
        std::printf(" %08x", bits((float)v));
    }
    std::printf("\nfp4_table");
    for (int n = 0; n < 16; n++) { std::printf(" %08x", bits(cccc::fp4_e2m1::to_float((uint8_t)n))); }
    std::printf("\n");

    std::vector<uint32_t> probes;
    unsigned int u;
    while (std::scanf("%x", &u) == 1) { probes.push_back(u); }
    std::printf("probes");
    for (auto p : probes) { std::printf(" %08x", p); }
    std::printf("\ne5m2_encode");
    for (auto p : probes) { std::printf(" %02x", cccc::fp8_e5m2(fromBits(p)).bits); }
    std::printf("\ne4m3_encode");
    for (auto p : probes) { std::printf(" %02x", cccc::fp8_e4m3(fromBits(p)).bits); }
    std::printf("\nfp4_encode");
    for (auto p : probes) { std::printf(" %02x", cccc::fp4_e2m1::from_float(fromBits(p))); }
    std::printf("\nbf16_host");
    for (auto p : probes) { std::printf(" %04x", cccc::bfloat16(fromBits(p)).bits); }
    std::printf("\n");

    // fp4 pack helpers: set() then get() on a small buffer
    uint8_t buf[8] = { 0 };
    const float vals[16] = { 0.f, 0.5f, -0.5f, 1.f, -1.5f, 2.f, 3.f, -4.f, 6.f, -6.f, 0.2f, 0.3f, 5.f, 4.9f, -0.f, 100.f };
    for (int i = 0; i < 16; i++) { cccc::fp4_e2m1::set(buf, i, vals[i]); }
    std::printf("fp4_pack");
    for (int i = 0; i < 8; i++) { std::printf(" %02x", buf[i]); }
    std::printf("\nfp4_get");
    for (int i = 0; i < 16; i++) { std::printf(" %08x", bits(cccc::fp4_e2m1::get(buf, i))); }
    std::printf("\n");
    return 0;
}
