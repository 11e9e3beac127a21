// ek_b200.hpp -- C++ host side above the C ABI of ek_b200.h, with the names and the error
// behaviour of the Expert Kit worker (Rust, `ek-computation`) for this path.  Header-only; link
// against libek_b200.so.
//
//   ek::EKError          <- EKError / EKResult            ek-base/src/error.rs:13-72
//   ek::EKInstance       <- EKInstance{hidden, intermediate}   ek-computation/src/x.rs:27-43
//   ek::ExpertDB         <- ExpertDB (mark_loading, insert, remove, has, loaded, loading, keys, load)
//                                                          ek-computation/src/worker/manager.rs:13-88
//   ek::ExpertBackend    <- ExpertBackend::build / forward    ek-computation/src/ffn/mod.rs:22-52
//   ek::ForwardReq/Resp  <- ek.worker.v1 ForwardReq / ForwardResp   ek-proto/ek/worker/v1/expert.proto:6-17
//   ek::EKInstanceGate   <- EKInstanceGate::forward           ek-computation/src/worker/core.rs:47-74
//
// Where the reference panics (empty request, sequences naming different experts: core.rs:52-57;
// a batch that is not 2-D: ffn/mod.rs:45) these throw EKError{InvalidInput} instead.
#ifndef EK_B200_HPP_
#define EK_B200_HPP_

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "ek_b200.h"

namespace ek {

class EKError : public std::runtime_error {
 public:
  EKError(int32_t status, const std::string& what)
      : std::runtime_error(std::string(ek_status_name(status)) + ": " + what), status_(status) {}
  int32_t status() const { return status_; }

 private:
  int32_t status_;
};

struct EKInstance {
  int32_t hidden = 0;
  int32_t intermediate = 0;
};

struct Sequence {
  std::vector<std::string> experts;
};
struct ForwardReq {
  std::string instance_id;
  std::vector<Sequence> sequences;
  std::vector<uint8_t> tensor;   // safetensors blob, single key "data", [n, H] BF16
};
struct ForwardResp {
  std::vector<uint8_t> output_tensor;   // same form
};

// The blob both directions carry (ek-computation/src/backend/torch/mod.rs:116;
// expertkit_torch/grpc_client.py:53,68-72).
inline std::vector<uint8_t> encode_data_blob(const void* bf16_rows, int64_t n, int64_t hidden) {
  const uint64_t bytes = (uint64_t)n * (uint64_t)hidden * 2;
  std::string hdr = "{\"data\":{\"dtype\":\"BF16\",\"shape\":[" + std::to_string(n) + "," + std::to_string(hidden) +
                    "],\"data_offsets\":[0," + std::to_string(bytes) + "]}}";
  while (hdr.size() % 8) hdr.push_back(' ');
  std::vector<uint8_t> out(8 + hdr.size() + bytes);
  const uint64_t hl = hdr.size();
  std::memcpy(out.data(), &hl, 8);   // little-endian hosts only, like the rest of the wire path
  std::memcpy(out.data() + 8, hdr.data(), hdr.size());
  std::memcpy(out.data() + 8 + hdr.size(), bf16_rows, bytes);
  return out;
}
// Payload of a reply produced by this library: the bytes after the header.
inline const uint8_t* data_blob_payload(const std::vector<uint8_t>& blob, size_t* bytes) {
  if (blob.size() < 8) throw EKError(EK_SAFETENSOR, "blob shorter than its length prefix");
  uint64_t hl;
  std::memcpy(&hl, blob.data(), 8);
  if (8 + hl > blob.size()) throw EKError(EK_SAFETENSOR, "header length exceeds the blob");
  *bytes = blob.size() - 8 - (size_t)hl;
  return blob.data() + 8 + hl;
}

class ExpertDB;

// A registered expert: what ExpertDB::load hands to the gate.
class ExpertBackend {
 public:
  // TorchFFN::forward: y[n,H] = down(up(x) * silu(gate(x))), bf16 rows, host or device pointers
  void forward(const void* x_bf16, int32_t n, void* y_bf16) const;
  const std::string& id() const { return id_; }

 private:
  friend class ExpertDB;
  ExpertBackend(const ExpertDB* db, std::string id) : db_(db), id_(std::move(id)) {}
  const ExpertDB* db_;
  std::string id_;
};

class ExpertDB {
 public:
  explicit ExpertDB(const ek_config_t& cfg) {
    const int32_t st = ek_backend_create(&cfg, &be_);
    if (st != EK_OK) throw EKError(st, ek_create_error());
    instance_.hidden = cfg.hidden;
    instance_.intermediate = cfg.intermediate;
  }
  ~ExpertDB() { ek_backend_destroy(be_); }
  ExpertDB(const ExpertDB&) = delete;
  ExpertDB& operator=(const ExpertDB&) = delete;

  // load_expert_task (ek-computation/src/worker/x.rs:13-34): claim, build, insert
  bool mark_loading(const std::string& id) {
    int32_t fresh = 0;
    check(ek_expert_mark_loading(be_, id.c_str(), &fresh));
    return fresh != 0;
  }
  void insert(const std::string& id, const std::vector<ek_tensor_view_t>& tensors) {
    check(ek_expert_register(be_, id.c_str(), tensors.data(), (int32_t)tensors.size()));
  }
  void insert_safetensors(const std::string& id, const void* blob, size_t len) {
    check(ek_expert_register_safetensors(be_, id.c_str(), blob, len));
  }
  void remove(const std::string& id) { check(ek_expert_evict(be_, id.c_str())); }
  bool has(const std::string& id) const { return ek_expert_has(be_, id.c_str()) != 0; }
  int32_t loaded() const { return ek_expert_loaded(be_); }
  int32_t loading() const { return ek_expert_loading(be_); }
  std::vector<std::string> keys() const {
    size_t need = 0;
    ek_expert_keys(be_, nullptr, 0, &need);
    std::string buf(need + 1, '\0');
    check(ek_expert_keys(be_, &buf[0], buf.size(), &need));
    std::vector<std::string> out;
    size_t pos = 0;
    const std::string s(buf.c_str());
    while (pos < s.size()) {
      size_t nl = s.find('\n', pos);
      if (nl == std::string::npos) nl = s.size();
      if (nl > pos) out.push_back(s.substr(pos, nl - pos));
      pos = nl + 1;
    }
    return out;
  }
  // ExpertDB::load (manager.rs:76-84): Err(ExpertNotFound) when the id is absent
  ExpertBackend load(const std::string& id) const {
    if (!has(id)) throw EKError(EK_EXPERT_NOT_FOUND, id);
    return ExpertBackend(this, id);
  }
  const EKInstance& instance() const { return instance_; }
  ek_backend_t* handle() const { return be_; }
  void check(int32_t st) const {
    if (st != EK_OK) throw EKError(st, ek_last_error(be_));
  }

 private:
  ek_backend_t* be_ = nullptr;
  EKInstance instance_;
};

inline void ExpertBackend::forward(const void* x_bf16, int32_t n, void* y_bf16) const {
  db_->check(ek_expert_forward(db_->handle(), id_.c_str(), x_bf16, n, y_bf16));
}

// The worker's request handler.  Safe to call from many threads at once: requests that arrive
// together are served as one grouped launch inside the library.
class EKInstanceGate {
 public:
  explicit EKInstanceGate(ExpertDB* db) : db_(db) {}
  ForwardResp forward(const ForwardReq& req) const {
    if (req.sequences.empty()) throw EKError(EK_INVALID_INPUT, "request without sequences");
    if (req.sequences[0].experts.size() != 1) throw EKError(EK_INVALID_INPUT, "a worker request names one expert per sequence");
    const std::string& id = req.sequences[0].experts[0];
    for (const Sequence& s : req.sequences)
      if (s.experts.size() != 1 || s.experts[0] != id)
        throw EKError(EK_INVALID_INPUT, "all sequences of a worker request must name the same expert");
    ForwardResp resp;
    size_t need = 0;
    resp.output_tensor.resize(req.tensor.size() + 64);
    int32_t st = ek_worker_forward_wire(db_->handle(), id.c_str(), req.tensor.data(), req.tensor.size(),
                                        resp.output_tensor.data(), resp.output_tensor.size(), &need);
    if (st == EK_INVALID_INPUT && need > resp.output_tensor.size()) {
      resp.output_tensor.resize(need);
      st = ek_worker_forward_wire(db_->handle(), id.c_str(), req.tensor.data(), req.tensor.size(),
                                  resp.output_tensor.data(), resp.output_tensor.size(), &need);
    }
    db_->check(st);
    resp.output_tensor.resize(need);
    return resp;
  }

 private:
  ExpertDB* db_;
};

}  // namespace ek

#endif  // EK_B200_HPP_
