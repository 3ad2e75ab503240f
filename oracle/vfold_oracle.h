/*
 * vfold_oracle.h — CPU oracle for the constant-folding path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain host restatement of the reference
 * compiler's fold arithmetic, used as the checker in tests/, in the smoke
 * check and as the timed CPU baseline of the benchmark. Nothing in the
 * product library links, loads or calls it.
 *
 * Parity pin: the restatement is checked against the reference's own unit
 * test vectors (tests/reference_cases.py, transcribed from
 * tests/unit/vpux_compiler/dialect/const/content_tests.cpp and the lit
 * weights-table goldens) and, for the fp16/bf16 converters, against the
 * reference's float16.cpp / bfloat16.cpp compiled unmodified into
 * oracle/_ref/libvpux_ref_types.so. Per-group u4 quantization and the
 * quantized-input bias column of the weights table have no reference test
 * vector: for those two, parity is defined by this restatement alone
 * ("parity unpinned").
 *
 * The entry points take the same POD descriptors as include/vfold.h so a test
 * can hand identical inputs to both sides.
 */
#ifndef VFOLD_ORACLE_H_
#define VFOLD_ORACLE_H_

#include "../include/vfold.h"

#ifdef __cplusplus
extern "C" {
#endif

/* element converters (bit patterns in, bit patterns out) */
uint16_t orc_f32_to_f16(uint32_t f32_bits);
uint32_t orc_f16_to_f32(uint16_t f16_bits);
uint16_t orc_f32_to_bf16(uint32_t f32_bits);
uint32_t orc_bf16_to_f32(uint16_t bf16_bits);
/* CvtHelper<float16>::cvt: RNE + clamp of infinities to +-65504 */
uint16_t orc_f32_to_f16_clamped(uint32_t f32_bits);
void orc_f32_to_f16_n(const uint32_t* in, uint16_t* out, uint64_t n);
void orc_f32_to_bf16_n(const uint32_t* in, uint16_t* out, uint64_t n);

int orc_calc_scale_zp(double qmin, double qmax, double rmin, double rmax, double* scale, int64_t* zp);
float orc_fake_quantize(float v, float in_low, float in_high, float q_low, float q_high, float levels);
int64_t orc_quantize_value(float x, double scale, int64_t zp, int64_t qmin, int64_t qmax);
float orc_dequantize_value(int64_t q, double scale, int64_t zp);
/* approximate<int32>(15, target) + arch37xx::getScale packing; returns status */
int orc_mult_shift(double rescale, int32_t* word, int32_t* mult, int32_t* shift);

/* `nthreads` selects the loop_nd-style partitioning used by the transformations the reference
 * parallelises; 1 = sequential. */
int orc_infer_type(const vf_tensor_type* base, int base_is_splat, const vf_transform* t, int n, vf_tensor_type* out,
                   int* out_is_splat, double* scales_buf, int64_t* zps_buf, int64_t params_cap, uint64_t* out_bytes,
                   char* err, size_t errlen);
int orc_fold(const vf_content* base, const vf_transform* t, int n, void* dst, uint64_t dst_bytes,
             uint64_t* dst_written, vf_tensor_type* out_type, double* scales_buf, int64_t* zps_buf,
             int64_t params_cap, int nthreads, char* err, size_t errlen);
int orc_row_stats(const vf_content* base, const vf_quant_spec* spec, double* scales, int64_t* zps, float* rmin,
                  float* rmax, int64_t n_units, int nthreads, char* err, size_t errlen);
int orc_quantize_fold(const vf_content* base, const vf_quant_spec* spec, const vf_transform* t, int n, void* dst,
                      uint64_t dst_bytes, uint64_t* dst_written, const vf_quant_outputs* outs, int nthreads,
                      char* err, size_t errlen);
int orc_nnz_per_oc(const vf_content* content, int64_t* counts, int nthreads, char* err, size_t errlen);
int orc_sparsify(const vf_content* content, void* data, uint64_t data_bytes, uint64_t* data_written, void* map,
                 uint64_t map_bytes, int64_t* counts, int nthreads, char* err, size_t errlen);
int orc_weights_table(const vf_weights_table_desc* desc, int32_t* table, int nthreads, char* err, size_t errlen);
int orc_synth_fill(const vf_synth_spec* spec, void* dst, uint64_t count, int nthreads);

#ifdef __cplusplus
}
#endif
#endif
