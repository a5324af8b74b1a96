// "TNNG" graph-state files: structure + layer configs + parameters of a graph
// (or of one pipeline stage). Byte layout, all little-endian, size_t = u64
// (reference writer/loader: src/nn/graph.cpp:422-692; tensor records:
// include/tensor/tensor_ops.hpp:17-66):
//
//   'T','N','N','G' | u32 version (2; 1 is read: inputs/outputs inferred)
//   u64 n_nodes   ; n x { u64 len ; bytes uid }
//   u64 n_inputs  ; n x u64 node index          (version >= 2)
//   u64 n_outputs ; n x u64 node index          (version >= 2)
//   u64 n_layers  ; n x { u64 len ; bytes json }   TConfig text of each unique layer
//   u64 n_edges   ; n x { u64 layer ; u64 np ; np x u64 ; u64 nc ; nc x u64 }
//   u64 n_layers  ; n x { u64 n_params ; n_params x TENSOR }
//   TENSOR = u32 dtype ; u64 ndim ; ndim x u64 ; raw row-major bytes
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "bytes.h"
#include "dtype.h"
#include "graph_ir.h"

namespace tnnb {

struct HostTensor {
  DType dtype = DType::FP32;
  std::vector<uint64_t> shape;
  std::string data;  // raw bytes, row-major
  uint64_t numel() const {
    uint64_t n = 1;
    for (uint64_t d : shape) n *= d;
    return n;
  }
};

void write_tensor(ByteWriter& w, const HostTensor& t);
HostTensor read_tensor(ByteReader& r);

struct GraphState {
  uint32_t version = 2;
  GraphIR ir;
  std::vector<std::string> layer_json;
  std::vector<std::vector<HostTensor>> params;  // per layer, descriptor order
};

std::string tnng_serialize(const GraphState& st);
GraphState tnng_parse(const char* data, size_t size);
void tnng_write_file(const std::string& path, const GraphState& st);
GraphState tnng_read_file(const std::string& path);

}  // namespace tnnb
