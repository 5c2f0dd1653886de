// The opaque handle types of include/oxb200.h, shared by the translation units that implement the C ABI.
#pragma once

#include "runtime.hpp"

struct oxb200_ctx {
  oxb::Context impl;
  oxb200_ctx(int device, const oxb200_config& cfg) : impl(device, cfg) {}
};
struct oxb200_tensor {
  oxb::DeviceTensorHandle h;
};
