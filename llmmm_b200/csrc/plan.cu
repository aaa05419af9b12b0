// Introspection and tuning behind the C ABI: what a call with given sizes would run (llmmm_describe_plan), and
// llmmm_tune, the tune(N, K) member the reference declares for its planned functor (src/mm/fp32/impl.h:20): the
// one-time per-device set-up a first call would otherwise pay, plus, for the FP8 kinds, a timed search over the
// plans of the decode-sized kernel for that weight shape.
#include "host_common.h"

extern "C" {

int llmmm_describe_plan(int kind, int M, int N, int K, char* buf, size_t len)
{
  using namespace llmmm;
  if (buf == nullptr || len == 0) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  buf[0] = '\0';
  const bool fp16 = kind == LLMMM_KIND_FP16 || kind == LLMMM_KIND_BF16;
  const bool fp8  = kind == LLMMM_KIND_FP8_E4M3OUT || kind == LLMMM_KIND_FP8_F32OUT;
  if (!fp16 && !fp8) {
    return set_error(LLMMM_ERR_UNSUPPORTED, "T is not supported. (kind %d)", kind);
  }
  if (fp16 && (M < 1 || N < 8 || K < 8 || (N % 8) != 0 || (K % 8) != 0)) {
    return set_error(LLMMM_ERR_SHAPE, "M or N or K are not aligned. (need M>=1, N%%8==0, K%%8==0; got %d %d %d)", M, N, K);
  }
  if (fp8 && (M < 1 || N < 128 || K < 128 || (N % 128) != 0 || (K % 128) != 0)) {
    return set_error(LLMMM_ERR_SHAPE, "M or N or K are not aligned. (need M>=1, N%%128==0, K%%128==0; got %d %d %d)", M, N, K);
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  if (fp16) {
    describe_fp16_plan(info, kind == LLMMM_KIND_BF16, M, N, K, buf, len);
  }
  else {
    describe_fp8_plan(info, kind == LLMMM_KIND_FP8_F32OUT, M, N, K, buf, len);
  }
  return LLMMM_OK;
}

int llmmm_tune(int kind, int N, int K)
{
  using namespace llmmm;
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  if (kind == LLMMM_KIND_FP16 || kind == LLMMM_KIND_BF16) {
    return warm_fp16_kernels(info);
  }
  if (kind == LLMMM_KIND_FP8_E4M3OUT || kind == LLMMM_KIND_FP8_F32OUT) {
    const int rc = warm_fp8_kernels(info);
    return rc != LLMMM_OK ? rc : tune_decode(info, N, K);
  }
  return set_error(LLMMM_ERR_UNSUPPORTED, "T is not supported. (kind %d)", kind);
}

}  // extern "C"
