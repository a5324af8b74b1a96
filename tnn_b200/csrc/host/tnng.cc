#include "tnng.h"

#include <fstream>
#include <sstream>

namespace tnnb {

void write_tensor(ByteWriter& w, const HostTensor& t) {
  if (t.data.size() != t.numel() * dtype_size(t.dtype)) throw std::runtime_error("tensor byte count does not match its shape");
  w.put<uint32_t>(static_cast<uint32_t>(t.dtype));
  w.put<uint64_t>(t.shape.size());
  for (uint64_t d : t.shape) w.put<uint64_t>(d);
  w.raw(t.data.data(), t.data.size());
}

HostTensor read_tensor(ByteReader& r) {
  HostTensor t;
  t.dtype = static_cast<DType>(r.get<uint32_t>());
  const uint64_t nd = r.get<uint64_t>();
  if (nd > 16) throw std::runtime_error("tensor record with more than 16 dimensions");
  t.shape.resize(nd);
  for (auto& d : t.shape) d = r.get<uint64_t>();
  const uint64_t bytes = t.numel() * dtype_size(t.dtype);
  t.data.assign(r.take(bytes), bytes);
  return t;
}

std::string tnng_serialize(const GraphState& st) {
  ByteWriter w;
  w.raw("TNNG", 4);
  w.put<uint32_t>(2);
  const GraphIR& g = st.ir;
  w.put<uint64_t>(g.nodes.size());
  for (const auto& uid : g.nodes) w.str(uid);
  w.put<uint64_t>(g.inputs.size());
  for (uint64_t i : g.inputs) w.put<uint64_t>(i);
  w.put<uint64_t>(g.outputs.size());
  for (uint64_t i : g.outputs) w.put<uint64_t>(i);
  w.put<uint64_t>(st.layer_json.size());
  for (const auto& s : st.layer_json) w.str(s);
  w.put<uint64_t>(g.edges.size());
  for (const auto& e : g.edges) {
    if (e.layer >= st.layer_json.size()) throw std::runtime_error("edge refers to a layer that is not in the state");
    w.put<uint64_t>(e.layer);
    w.put<uint64_t>(e.producers.size());
    for (uint64_t p : e.producers) w.put<uint64_t>(p);
    w.put<uint64_t>(e.consumers.size());
    for (uint64_t c : e.consumers) w.put<uint64_t>(c);
  }
  if (st.params.size() != st.layer_json.size()) throw std::runtime_error("parameter section does not match layer count");
  w.put<uint64_t>(st.params.size());
  for (const auto& lp : st.params) {
    w.put<uint64_t>(lp.size());
    for (const auto& t : lp) write_tensor(w, t);
  }
  return std::move(w.buf);
}

GraphState tnng_parse(const char* data, size_t size) {
  ByteReader r(data, size);
  const char* magic = r.take(4);
  if (std::string(magic, 4) != "TNNG") throw std::runtime_error("Invalid graph state file header");
  GraphState st;
  st.version = r.get<uint32_t>();
  if (st.version != 1 && st.version != 2) throw std::runtime_error("Unsupported graph state version: " + std::to_string(st.version));
  GraphIR& g = st.ir;
  const uint64_t nn = r.get<uint64_t>();
  for (uint64_t i = 0; i < nn; ++i) g.add_node(r.str());
  auto read_index_set = [&](std::vector<uint64_t>& dst, const char* what) {
    const uint64_t n = r.get<uint64_t>();
    for (uint64_t i = 0; i < n; ++i) {
      const uint64_t idx = r.get<uint64_t>();
      if (idx >= nn) throw std::runtime_error(std::string("Graph state references an invalid ") + what + " node index");
      dst.push_back(idx);
    }
  };
  if (st.version >= 2) {
    read_index_set(g.inputs, "input");
    read_index_set(g.outputs, "output");
  }
  const uint64_t nl = r.get<uint64_t>();
  for (uint64_t i = 0; i < nl; ++i) st.layer_json.push_back(r.str());
  const uint64_t ne = r.get<uint64_t>();
  for (uint64_t i = 0; i < ne; ++i) {
    IrEdge e;
    e.layer = r.get<uint64_t>();
    if (e.layer >= nl) throw std::runtime_error("Graph state references an invalid layer index");
    const uint64_t np = r.get<uint64_t>();
    for (uint64_t k = 0; k < np; ++k) {
      const uint64_t idx = r.get<uint64_t>();
      if (idx >= nn) throw std::runtime_error("Graph state references an invalid producer node index");
      e.producers.push_back(idx);
    }
    const uint64_t nc = r.get<uint64_t>();
    for (uint64_t k = 0; k < nc; ++k) {
      const uint64_t idx = r.get<uint64_t>();
      if (idx >= nn) throw std::runtime_error("Graph state references an invalid consumer node index");
      e.consumers.push_back(idx);
    }
    g.edges.push_back(std::move(e));
  }
  if (st.version == 1) {
    for (uint64_t n = 0; n < nn; ++n) {
      if (g.in_degree(n) == 0) g.inputs.push_back(n);
      if (g.out_degree(n) == 0) g.outputs.push_back(n);
    }
  }
  const uint64_t npl = r.get<uint64_t>();
  if (npl != nl) throw std::runtime_error("Graph state parameter section does not match layer count");
  st.params.resize(nl);
  for (uint64_t i = 0; i < nl; ++i) {
    const uint64_t np = r.get<uint64_t>();
    for (uint64_t k = 0; k < np; ++k) st.params[i].push_back(read_tensor(r));
  }
  return st;
}

void tnng_write_file(const std::string& path, const GraphState& st) {
  const std::string bytes = tnng_serialize(st);
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  if (!f) throw std::runtime_error("cannot open for writing: " + path);
  f.write(bytes.data(), static_cast<std::streamsize>(bytes.size()));
  if (!f) throw std::runtime_error("Failed to write graph state: " + path);
}

GraphState tnng_read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open for reading: " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string bytes = ss.str();
  return tnng_parse(bytes.data(), bytes.size());
}

}  // namespace tnnb
