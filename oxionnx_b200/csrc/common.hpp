// Shared host-side definitions of the oxb200 runtime.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/oxb200.h"

namespace oxb {

// Device storage type of a value.  The boundary speaks f32 lanes; on the device a value is
// stored in the narrowest type that holds every lane the reference can produce for it.
enum class DT : int32_t { F32 = 0, U8 = 1, I8 = 2, I32 = 3, I16 = 4, F16 = 5, BF16 = 6 };

inline size_t dt_size(DT d) {
  switch (d) {
    case DT::F32: return 4;
    case DT::U8: return 1;
    case DT::I8: return 1;
    case DT::I32: return 4;
    case DT::I16: return 2;
    case DT::F16: return 2;
    case DT::BF16: return 2;
  }
  return 4;
}
inline const char* dt_name(DT d) {
  switch (d) {
    case DT::F32: return "f32";
    case DT::U8: return "u8";
    case DT::I8: return "i8";
    case DT::I32: return "i32";
    case DT::I16: return "i16";
    case DT::F16: return "f16";
    case DT::BF16: return "bf16";
  }
  return "?";
}

// Memory order of a device value.  PLAIN is row-major in the logical (ONNX) shape.  NHWC
// applies to rank-4 [N,C,H,W] values and stores them channels-last, which is what the TMA
// im2col loads and the GEMM-shaped epilogue stores want.
enum class Layout : int32_t { PLAIN = 0, NHWC = 1 };

struct Status {
  int code;  // OXB200_* outcome
  std::string message;
};

// Control-flow exception used inside the library only; abi.cpp converts it to a status.
struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

[[noreturn]] inline void raise(int code, const char* fmt, ...) {
  char buf[768];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  throw Error(code, buf);
}

#define OXB_DECLINE(...) ::oxb::raise(OXB200_DECLINED, __VA_ARGS__)
#define OXB_FAIL(...) ::oxb::raise(OXB200_FAILED, __VA_ARGS__)

#define OXB_CUDA(expr)                                                                                   \
  do {                                                                                                   \
    cudaError_t _e = (expr);                                                                             \
    if (_e != cudaSuccess) ::oxb::raise(OXB200_FAILED, "CUDA error %s at %s:%d: %s", cudaGetErrorName(_e), \
                                        __FILE__, __LINE__, cudaGetErrorString(_e));                     \
  } while (0)

// Records a message for oxb200_last_error(NULL) on the calling thread (defined in abi.cpp).
void set_thread_error(const std::string& message);

inline int64_t prod(const std::vector<int64_t>& s) {
  int64_t n = 1;
  for (int64_t d : s) n *= d;
  return n;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

}  // namespace oxb
