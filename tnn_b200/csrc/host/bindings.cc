// pybind11 surface of the host runtime (module tnn_b200._lib._host).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "graph_ir.h"
#include "profiler.h"
#include "tconfig.h"
#include "tnng.h"
#include "tcp_comm.h"
#include "wire.h"

namespace py = pybind11;
using namespace tnnb;

namespace tnnb {
void bind_cpu_engine(py::module_& m);
void bind_runtime(py::module_& m);
}  // namespace tnnb

// Tensors cross the boundary as (dtype code, shape, bytes).
static py::tuple tensor_to_py(const HostTensor& t) {
  return py::make_tuple(static_cast<uint32_t>(t.dtype), t.shape, py::bytes(t.data));
}
static HostTensor tensor_from_py(const py::handle& h) {
  py::tuple t = py::cast<py::tuple>(h);
  HostTensor o;
  o.dtype = static_cast<DType>(t[0].cast<uint32_t>());
  o.shape = t[1].cast<std::vector<uint64_t>>();
  o.data = t[2].cast<std::string>();
  return o;
}

static GraphIR ir_from_py(const py::dict& d) {
  GraphIR g;
  for (auto uid : d["nodes"]) g.add_node(uid.cast<std::string>());
  g.inputs = d["inputs"].cast<std::vector<uint64_t>>();
  g.outputs = d["outputs"].cast<std::vector<uint64_t>>();
  for (auto e : d["edges"]) {
    py::tuple t = py::cast<py::tuple>(e);
    g.add_edge(t[0].cast<uint64_t>(), t[1].cast<std::vector<uint64_t>>(), t[2].cast<std::vector<uint64_t>>());
  }
  return g;
}
static py::dict ir_to_py(const GraphIR& g) {
  py::dict d;
  d["nodes"] = g.nodes;
  d["inputs"] = g.inputs;
  d["outputs"] = g.outputs;
  py::list edges;
  for (const auto& e : g.edges) edges.append(py::make_tuple(e.layer, e.producers, e.consumers));
  d["edges"] = edges;
  return d;
}

static GraphState state_from_py(const py::dict& d) {
  GraphState st;
  st.ir = ir_from_py(d);
  st.layer_json = d["layers"].cast<std::vector<std::string>>();
  for (auto lp : d["params"]) {
    std::vector<HostTensor> v;
    for (auto t : lp) v.push_back(tensor_from_py(t));
    st.params.push_back(std::move(v));
  }
  return st;
}
static py::dict state_to_py(const GraphState& st) {
  py::dict d = ir_to_py(st.ir);
  d["version"] = st.version;
  d["layers"] = st.layer_json;
  py::list params;
  for (const auto& lp : st.params) {
    py::list l;
    for (const auto& t : lp) l.append(tensor_to_py(t));
    params.append(l);
  }
  d["params"] = params;
  return d;
}

static Message message_from_py(const py::dict& d) {
  Message m;
  m.command = d["command"].cast<uint16_t>();
  m.kind = d.contains("kind") ? d["kind"].cast<uint32_t>() : 0u;
  if (m.kind == PAYLOAD_JOB) {
    py::dict j = d["job"];
    m.job.pid = j["pid"].cast<uint64_t>();
    for (auto kv : j["tensors"]) {
      py::tuple t = py::cast<py::tuple>(kv);
      m.job.tensors.emplace_back(t[0].cast<std::string>(), tensor_from_py(t[1]));
    }
  } else if (m.kind == PAYLOAD_STRING) {
    m.text = d["text"].cast<std::string>();
  } else if (m.kind == PAYLOAD_BOOL) {
    m.flag = d["flag"].cast<bool>();
  } else if (m.kind == PAYLOAD_PROFILER) {
    py::dict p = d["profiler"];
    m.profiler.start_time = p["start_time"].cast<int64_t>();
    for (auto ev : p["events"]) {
      py::tuple t = py::cast<py::tuple>(ev);
      m.profiler.events.push_back({t[0].cast<int64_t>(), t[1].cast<int64_t>(), t[2].cast<uint8_t>(), t[3].cast<std::string>(), t[4].cast<std::string>()});
    }
  } else if (m.kind == PAYLOAD_STAGE_CONFIG) {
    py::dict s = d["stage"];
    m.stage.graph_state = s["graph_state"].cast<std::string>();
    m.stage.input_uids = s["input_uids"].cast<std::vector<std::string>>();
    m.stage.output_uids = s["output_uids"].cast<std::vector<std::string>>();
    m.stage.optimizer_config = s["optimizer_config"].cast<std::string>();
    m.stage.scheduler_config = s["scheduler_config"].cast<std::string>();
    m.stage.next_stage = s["next_stage"].cast<std::string>();
    m.stage.prev_stage = s["prev_stage"].cast<std::string>();
    m.stage.coordinator = s["coordinator"].cast<std::string>();
  }
  return m;
}
static py::dict message_to_py(const Message& m) {
  py::dict d;
  d["command"] = m.command;
  d["command_name"] = command_name(m.command);
  d["kind"] = m.kind;
  if (m.kind == PAYLOAD_JOB) {
    py::dict j;
    j["pid"] = m.job.pid;
    py::list ts;
    for (const auto& kv : m.job.tensors) ts.append(py::make_tuple(kv.first, tensor_to_py(kv.second)));
    j["tensors"] = ts;
    d["job"] = j;
  } else if (m.kind == PAYLOAD_STRING) {
    d["text"] = m.text;
  } else if (m.kind == PAYLOAD_BOOL) {
    d["flag"] = m.flag;
  } else if (m.kind == PAYLOAD_PROFILER) {
    py::dict p;
    p["start_time"] = m.profiler.start_time;
    py::list evs;
    for (const auto& e : m.profiler.events) evs.append(py::make_tuple(e.start, e.end, e.type, e.name, e.source));
    p["events"] = evs;
    d["profiler"] = p;
  } else if (m.kind == PAYLOAD_STAGE_CONFIG) {
    py::dict s;
    s["graph_state"] = py::bytes(m.stage.graph_state);
    s["input_uids"] = m.stage.input_uids;
    s["output_uids"] = m.stage.output_uids;
    s["optimizer_config"] = m.stage.optimizer_config;
    s["scheduler_config"] = m.stage.scheduler_config;
    s["next_stage"] = m.stage.next_stage;
    s["prev_stage"] = m.stage.prev_stage;
    s["coordinator"] = m.stage.coordinator;
    d["stage"] = s;
  }
  return d;
}

PYBIND11_MODULE(_host, m) {
  m.doc() = "tnn_b200 host runtime: typed config, TNNG checkpoints, wire format, graph IR, partitioner, profiler";

  // ---- dtype ----
  m.def("dtype_size", [](uint32_t c) { return dtype_size(static_cast<DType>(c)); });
  m.def("dtype_name", [](uint32_t c) { return std::string(dtype_name(static_cast<DType>(c))); });
  m.def("dtype_code", [](const std::string& s) { return static_cast<uint32_t>(dtype_from_name(s)); });
  m.def("f32_to_bf16", &f32_to_bf16);
  m.def("bf16_to_f32", &bf16_to_f32);

  // ---- TConfig ----
  py::class_<TConfig>(m, "TConfig")
      .def(py::init<>())
      .def_readwrite("name", &TConfig::name)
      .def_readwrite("type", &TConfig::type)
      .def("set", [](TConfig& c, const std::string& k, const std::string& tag, py::object v) {
        py::module_ json = py::module_::import("json");
        c.set_tagged(k, tag, Json::parse(json.attr("dumps")(v).cast<std::string>()));
      })
      .def("has", &TConfig::has)
      .def("remove", &TConfig::remove)
      .def("tag", [](const TConfig& c, const std::string& k) { return c.at(k).tag; })
      .def("get", [](const TConfig& c, const std::string& k) {
        py::module_ json = py::module_::import("json");
        return json.attr("loads")(c.at(k).value.dump());
      })
      .def("keys", [](const TConfig& c) {
        std::vector<std::string> ks;
        for (const auto& kv : c.parameters()) ks.push_back(kv.first);
        return ks;
      })
      .def("dump", &TConfig::dump)
      .def_static("parse", &TConfig::parse);
  m.def("tconfig_normalize", [](const std::string& text) { return TConfig::parse(text).dump(); },
        "parse a TConfig JSON text and re-emit it in canonical (key-sorted, compact, typed) form");

  // ---- graph IR / partitioner ----
  m.def("topo_sort", [](const py::dict& d) {
    GraphIR g = ir_from_py(d);
    std::vector<uint64_t> node_perm;
    std::vector<uint64_t> edge_perm = g.sort(&node_perm);
    py::dict out = ir_to_py(g);
    out["edge_perm"] = edge_perm;
    out["node_perm"] = node_perm;
    return out;
  }, "FIFO Kahn sort; returns the reordered graph plus edge_perm / node_perm (new -> old)");
  m.def("resolve_layer_counts", &resolve_layer_counts);
  m.def("partition", [](const py::dict& d, const std::vector<double>& ratios) {
    GraphIR g = ir_from_py(d);
    py::list out;
    for (const auto& p : partition_graph(g, ratios)) {
      py::dict pd = ir_to_py(p.graph);
      pd["input_uids"] = p.input_uids;
      pd["output_uids"] = p.output_uids;
      pd["start_layer"] = p.start_layer;
      pd["layer_count"] = p.layer_count;
      pd["edge_ids"] = p.edge_ids;
      out.append(pd);
    }
    return out;
  });

  // ---- TNNG ----
  m.def("tnng_serialize", [](const py::dict& d) { return py::bytes(tnng_serialize(state_from_py(d))); });
  m.def("tnng_parse", [](const std::string& b) { return state_to_py(tnng_parse(b.data(), b.size())); });
  m.def("tnng_write_file", [](const std::string& path, const py::dict& d) { tnng_write_file(path, state_from_py(d)); });
  m.def("tnng_read_file", [](const std::string& path) { return state_to_py(tnng_read_file(path)); });
  m.def("tensor_serialize", [](py::tuple t) {
    ByteWriter w;
    write_tensor(w, tensor_from_py(t));
    return py::bytes(w.buf);
  });
  m.def("tensor_parse", [](const std::string& b) {
    ByteReader r(b.data(), b.size());
    return tensor_to_py(read_tensor(r));
  });

  // ---- wire ----
  m.attr("PACKET_HEADER_SIZE") = PacketHeader::kSize;
  m.def("command_name", &command_name);
  m.def("command_code", [](const std::string& s) {
    for (uint16_t i = 0; i < CMD_COUNT; ++i)
      if (s == command_name(i)) return static_cast<int>(i);
    return -1;
  });
  m.def("serialize_message", [](const py::dict& d) { return py::bytes(serialize_message(message_from_py(d))); });
  m.def("parse_message", [](const std::string& b, bool swap) { return message_to_py(parse_message(b.data(), b.size(), swap)); },
        py::arg("data"), py::arg("swap_endian") = false);
  m.def("slice_message", [](const std::string& b, uint64_t id, uint64_t max_packet) {
    py::list out;
    for (auto& p : slice_message(b, id, max_packet)) out.append(py::bytes(p));
    return out;
  });
  m.def("parse_packet_header", [](const std::string& b) {
    PacketHeader h = read_packet_header(b.data(), b.size());
    py::dict d;
    d["version"] = h.version; d["type"] = h.type; d["little_endian"] = h.little_endian;
    d["packet_length"] = h.packet_length; d["msg_length"] = h.msg_length; d["msg_serial_id"] = h.msg_serial_id;
    d["packet_offset"] = h.packet_offset; d["total_packets"] = h.total_packets; d["compression"] = h.compression;
    return d;
  });
  py::class_<Aggregator>(m, "Aggregator")
      .def(py::init<uint64_t, uint32_t>(), py::arg("max_message_bytes") = 16ull << 30, py::arg("max_packets") = 1u << 22)
      .def("feed", [](Aggregator& a, const std::string& pkt) -> py::object {
        std::string out;
        uint64_t id = 0;
        if (a.feed(pkt.data(), pkt.size(), &out, &id)) return py::make_tuple(id, py::bytes(out));
        return py::none();
      })
      .def("pending", &Aggregator::pending);

  // ---- TCP transport (blocking calls release the interpreter lock) ----
  // The destructor joins writer threads that may be waiting for the interpreter lock to release a bytes object,
  // so the lock is dropped while the communicator is destroyed.
  struct TcpDeleter {
    void operator()(TcpCommunicator* p) const {
      py::gil_scoped_release rel;
      delete p;
    }
  };
  py::class_<TcpCommunicator, std::unique_ptr<TcpCommunicator, TcpDeleter>>(m, "TcpCommunicator")
      .def(py::init<std::string, int, int, uint64_t>(), py::arg("host") = "127.0.0.1", py::arg("port") = 0,
           py::arg("sockets_per_endpoint") = 4, py::arg("max_packet_size") = 4ull << 20)
      .def("start", &TcpCommunicator::start, py::call_guard<py::gil_scoped_release>())
      .def("set_max_message_bytes", &TcpCommunicator::set_max_message_bytes)
      .def("endpoint", &TcpCommunicator::endpoint)
      .def("connect", &TcpCommunicator::connect, py::arg("host"), py::arg("port"), py::arg("timeout_s") = 10.0,
           py::call_guard<py::gil_scoped_release>())
      .def("connected", &TcpCommunicator::connected)
      .def("peers", &TcpCommunicator::peers)
      .def("send", [](TcpCommunicator& c, const std::string& ep, const py::bytes& data) {
        // no copy: the packets point into the bytes object, which is released (under the interpreter lock, from a
        // writer thread) after the last of them has been written
        char* p = nullptr;
        Py_ssize_t n = 0;
        if (PyBytes_AsStringAndSize(data.ptr(), &p, &n) != 0) throw py::error_already_set();
        PyObject* obj = data.ptr();
        Py_INCREF(obj);
        std::shared_ptr<const void> keep(static_cast<const void*>(obj), [](const void* o) {
          py::gil_scoped_acquire g;
          Py_DECREF(reinterpret_cast<PyObject*>(const_cast<void*>(o)));
        });
        py::gil_scoped_release rel;
        c.send_view(ep, p, static_cast<size_t>(n), std::move(keep));
      })
      .def("recv", [](TcpCommunicator& c, double timeout_s) -> py::object {
        std::string ep, msg;
        bool ok;
        {
          py::gil_scoped_release rel;
          ok = c.recv(timeout_s, &ep, &msg);
        }
        if (!ok) return py::none();
        return py::make_tuple(ep, py::bytes(msg));
      }, py::arg("timeout_s") = -1.0)
      .def("echo", [](TcpCommunicator& c, const std::string& stop) {
        py::gil_scoped_release rel;
        return c.echo(stop);
      }, py::arg("stop_message"))
      .def("ping_pong", [](TcpCommunicator& c, const std::string& ep, size_t bytes, double seconds) {
        double dt = 0.0;
        uint64_t n;
        {
          py::gil_scoped_release rel;
          n = c.ping_pong(ep, bytes, seconds, &dt);
        }
        return py::make_tuple(n, dt);
      }, py::arg("endpoint"), py::arg("message_bytes"), py::arg("seconds"))
      .def("flush", &TcpCommunicator::flush, py::arg("timeout_s") = 30.0, py::call_guard<py::gil_scoped_release>())
      .def("stop", &TcpCommunicator::stop, py::call_guard<py::gil_scoped_release>())
      .def("stats", [](const TcpCommunicator& c) {
        py::dict d;
        d["bytes_sent"] = c.bytes_sent(); d["bytes_received"] = c.bytes_received();
        d["messages_sent"] = c.messages_sent(); d["messages_received"] = c.messages_received();
        return d;
      });

  // ---- profiler ----
  py::class_<Profiler>(m, "Profiler")
      .def(py::init<>())
      .def("start", &Profiler::start)
      .def("start_time", &Profiler::start_time)
      .def("set_start_time", &Profiler::set_start_time)
      .def("add_event", &Profiler::add_event, py::arg("type"), py::arg("start_ns"), py::arg("end_ns"), py::arg("name"), py::arg("source"))
      .def("clear", &Profiler::clear)
      .def("__len__", &Profiler::size)
      .def("merge", &Profiler::merge)
      .def("sort", &Profiler::sort)
      .def("log_lines", &Profiler::log_lines)
      .def("events", [](const Profiler& p) {
        py::list l;
        for (const auto& e : p.events()) l.append(py::make_tuple(e.start, e.end, e.type, e.name, e.source));
        return l;
      })
      .def("to_message_dict", [](const Profiler& p) {
        Message msg;
        msg.command = PROFILING_REPORTED;
        msg.kind = PAYLOAD_PROFILER;
        msg.profiler = p.data();
        return message_to_py(msg);
      })
      .def_static("from_message_dict", [](const py::dict& d) { return Profiler::from_data(message_from_py(d).profiler); })
      .def_static("now_ns", &Profiler::now_ns);

  bind_cpu_engine(m);
  bind_runtime(m);
}
