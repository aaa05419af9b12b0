/* C declarations of the CPU oracle (oracle.cpp).  TEST INFRASTRUCTURE ONLY:
 * included by the harness drivers under tests/, never by the product library. */
#ifndef LLMMM_ORACLE_H
#define LLMMM_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
int  oracle_num_threads(void);
void oracle_e4m3_decode(const uint8_t* q, float* out, int64_t n);
void oracle_f32_to_f16(const float* x, uint16_t* out, int64_t n);
void oracle_f16_to_f32(const uint16_t* x, float* out, int64_t n);
void oracle_kahan_gemm(const float* A, const float* B, float* C, int M, int N, int K, int row0, int rows);
void oracle_double_gemm(const float* A, const float* B, float* C, int M, int N, int K, int row0, int rows);
void oracle_exact_gemm_f64(const float* A, const float* B, double* C, int M, int N, int K, int row0, int rows);
void oracle_quant_1x128(const float* x, uint8_t* q, float* scale, int M, int K);
void oracle_quant_128x128(const float* x, uint8_t* q, float* scale, int rows, int cols);
void oracle_fp8_blockwise_acc(const uint8_t* A_q, const float* A_s, const uint8_t* B_q, const float* B_s,
                              float* acc_f32, double* acc_f64, int M, int N, int K, int row0, int rows, int mode);
void oracle_c_quant_1x128(const float* acc, uint8_t* C_q, float* C_s, int rows, int N, int ldcs, int row0);
void oracle_dequant_1x128(const uint8_t* q, const float* s, float* out, int M, int N);
#ifdef __cplusplus
}
#endif
#endif
