// An ONNX model as this provider sees it after loading: topologically sorted nodes, initializers as f32 lanes with
// their declared element types, graph inputs and outputs.  The loader restates what oxionnx-proto does for the
// parts of the format the hot path needs (src/reader.rs, src/parser.rs, src/types.rs, src/model.rs); the passes of
// optimize() restate the reference's Conv / InstanceNorm fusions (src/optimizer/fusion/conv/*.rs,
// src/optimizer/fusion/instance_norm.rs), which produce the fused-node contract the kernels implement.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "runtime.hpp"

namespace oxb {

struct ModelValueInfo {
  std::string name;
  std::vector<int64_t> shape;  // -1 for a symbolic or missing dimension
  int32_t onnx_dtype = 1;      // TensorProto.DataType
};

struct Model {
  std::vector<NodeDef> nodes;
  std::map<std::string, HostTensor> initializers;
  std::vector<std::string> initializer_order;  // file order, for stable listings
  std::vector<ModelValueInfo> inputs;          // graph inputs that are not initializers
  std::vector<ModelValueInfo> outputs;
  std::map<std::string, std::vector<int64_t>> known_shapes;  // value_info + inputs: rank information for the matchers
  int64_t ir_version = 0, opset = 0;
  std::string producer;
};

// Parses ModelProto bytes.  Throws Error(OXB200_FAILED) on malformed input, Error(OXB200_DECLINED) on features this
// provider does not take (external data, subgraph attributes, sparse initializers, non-numeric tensors).
Model load_onnx(const uint8_t* bytes, size_t len);

// The reference's fusion passes, in its order: MatMul+Add -> Gemm, Conv+BatchNormalization fold, Conv+Relu /
// Conv+Clip, Conv+Clip(0,6), Mul(x, Sigmoid(x)) -> SiLU, the InstanceNorm-style chain -> OxiInstanceNorm,
// Conv+Add+Relu -> ConvAddRelu.
// Returns how many nodes were removed.  level 0: nothing; 1: everything above.
int optimize_model(Model& m, int level);

// Individual passes (exposed for the known-answer tests that pin each against the reference's own).
int fuse_conv_batchnorm(Model& m);
int fuse_conv_relu(Model& m);
int fuse_conv_clip_to_relu6(Model& m);
int fuse_instance_norm(Model& m);
int fuse_matmul_add(Model& m);
int fuse_mul_sigmoid_to_silu(Model& m);
int fuse_conv_add_relu(Model& m);
// Puts the nodes back into a topological order (a fused node may have moved ahead of one of its inputs' producers).
void topo_sort(Model& m);

// Element type of this provider for an ONNX data type, or false when the boundary does not take it.
bool onnx_dtype_to_dt(int32_t onnx_dtype, DT* out);

}  // namespace oxb
