// C entry points around the reference's own float16 / bfloat16 classes. This file is compiled together with
// the reference's float16.cpp and bfloat16.cpp taken unmodified from the reference tree (see Makefile, target
// `ref`); it contains no arithmetic of its own. TEST INFRASTRUCTURE ONLY.
#include <cstdint>
#include <cstring>

#include <vpux/utils/core/type/bfloat16.hpp>
#include <vpux/utils/core/type/float16.hpp>

extern "C" {
uint16_t ref_f32_to_f16(uint32_t bits) {
    float f;
    std::memcpy(&f, &bits, 4);
    return vpux::type::float16(f).to_bits();
}
uint32_t ref_f16_to_f32(uint16_t h) {
    const float f = static_cast<float>(vpux::type::float16::from_bits(h));
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    return bits;
}
uint16_t ref_f32_to_bf16(uint32_t bits) {
    float f;
    std::memcpy(&f, &bits, 4);
    return vpux::type::bfloat16(f).to_bits();
}
uint32_t ref_bf16_to_f32(uint16_t h) {
    const float f = static_cast<float>(vpux::type::bfloat16::from_bits(h));
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    return bits;
}
// bulk forms so a test can sweep millions of patterns quickly
void ref_f32_to_f16_n(const uint32_t* in, uint16_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = ref_f32_to_f16(in[i]);
}
void ref_f32_to_bf16_n(const uint32_t* in, uint16_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = ref_f32_to_bf16(in[i]);
}
}
