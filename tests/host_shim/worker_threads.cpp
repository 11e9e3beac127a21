// Drives the C++ mirror of the worker (include/ek_b200.hpp) the way the reference's runtime does:
// one EKInstanceGate::forward per expert, from many threads at once
// (ek-computation/src/worker/core.rs:47-74, bin/worker.rs:5: 48 runtime threads).
//
//   worker_threads <hidden> <intermediate> <experts> <rows per call> <threads> <rounds>
//
// Registers `experts` random bf16 experts, runs every expert once from one thread (the answers),
// then `rounds` times from `threads` threads, compares the reply blobs byte for byte and prints one
// JSON line.  Exit codes: 0 ok, 2 mismatch or error, 3 no CUDA device (printed on stderr).
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <thread>

#include "ek_b200.hpp"

static uint32_t rng_state = 12345u;
static uint32_t rng() {
  rng_state ^= rng_state << 13;
  rng_state ^= rng_state >> 17;
  rng_state ^= rng_state << 5;
  return rng_state;
}
// roughly N(0, sigma): sum of four uniforms, as bf16 bits (truncation is fine for test data)
static uint16_t bf16_normal(float sigma) {
  float u = 0.f;
  for (int i = 0; i < 4; ++i) u += (float)(rng() & 0xFFFF) / 65536.0f - 0.5f;
  const float v = u * 1.7320508f * sigma;
  uint32_t bits;
  std::memcpy(&bits, &v, 4);
  return (uint16_t)(bits >> 16);
}

int main(int argc, char** argv) {
  if (argc < 7) {
    std::fprintf(stderr, "usage: %s hidden intermediate experts rows threads rounds\n", argv[0]);
    return 2;
  }
  const int H = std::atoi(argv[1]), I = std::atoi(argv[2]), E = std::atoi(argv[3]), n = std::atoi(argv[4]);
  const int n_threads = std::atoi(argv[5]), rounds = std::atoi(argv[6]);
  ek_config_t cfg;
  std::memset(&cfg, 0, sizeof cfg);
  cfg.hidden = H; cfg.intermediate = I; cfg.n_experts = E; cfg.top_k = 1; cfg.scoring = EK_SCORE_SOFTMAX;
  cfg.n_group = 1; cfg.topk_group = 1; cfg.norm_topk_prob = 1; cfg.routed_scaling = 1.f;
  cfg.quant = EK_QUANT_BF16; cfg.max_tokens = n * E; cfg.max_layers = 1; cfg.ep_size = 1;
  std::snprintf(cfg.model_name, sizeof cfg.model_name, "shim");
  try {
    ek::ExpertDB db(cfg);
    ek::EKInstanceGate gate(&db);
    std::vector<uint16_t> up((size_t)I * H), gatew((size_t)I * H), down((size_t)H * I);
    std::vector<std::string> ids;
    for (int e = 0; e < E; ++e) {
      for (auto& v : up) v = bf16_normal(0.02f);
      for (auto& v : gatew) v = bf16_normal(0.02f);
      for (auto& v : down) v = bf16_normal(0.02f);
      const std::string id = "shim/l0-e" + std::to_string(e);
      if (!db.mark_loading(id)) throw ek::EKError(EK_INVALID_INPUT, "id claimed twice");
      // names as the weight server delivers them; picked by suffix (ffn/meta.rs:57-75)
      std::vector<ek_tensor_view_t> t(3);
      const std::string base = "model.layers.0.mlp.experts." + std::to_string(e);
      const std::string n1 = base + ".w1.weight", n2 = base + ".w2.weight", n3 = base + ".w3.weight";
      t[0] = {n1.c_str(), EK_BF16, 2, {I, H, 0, 0}, up.data()};
      t[1] = {n2.c_str(), EK_BF16, 2, {H, I, 0, 0}, down.data()};
      t[2] = {n3.c_str(), EK_BF16, 2, {I, H, 0, 0}, gatew.data()};
      db.insert(id, t);
      ids.push_back(id);
    }
    if (db.loaded() != E || (int)db.keys().size() != E) throw ek::EKError(EK_INVALID_INPUT, "registry count is off");
    // one request per expert
    std::vector<ek::ForwardReq> reqs(E);
    std::vector<uint16_t> x((size_t)n * H);
    for (int e = 0; e < E; ++e) {
      for (auto& v : x) v = bf16_normal(1.0f);
      reqs[e].instance_id = "shim";
      reqs[e].sequences.assign(n, ek::Sequence{{ids[e]}});
      reqs[e].tensor = ek::encode_data_blob(x.data(), n, H);
    }
    int64_t c0 = 0, b0 = 0, c1 = 0, b1 = 0, c2 = 0, b2 = 0;
    db.check(ek_worker_batch_stats(db.handle(), &c0, &b0));
    std::vector<ek::ForwardResp> want(E);
    for (int e = 0; e < E; ++e) want[e] = gate.forward(reqs[e]);   // warm-up + answers
    auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < rounds; ++r)
      for (int e = 0; e < E; ++e) gate.forward(reqs[e]);
    const double seq_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / rounds;
    db.check(ek_worker_batch_stats(db.handle(), &c1, &b1));
    std::atomic<int> mismatches{0}, errors{0};
    t0 = std::chrono::steady_clock::now();
    std::vector<std::thread> ths;
    for (int t = 0; t < n_threads; ++t)
      ths.emplace_back([&, t] {
        try {
          for (int r = 0; r < rounds; ++r)
            for (int e = t; e < E; e += n_threads) {
              const ek::ForwardResp got = gate.forward(reqs[e]);
              if (got.output_tensor != want[e].output_tensor) ++mismatches;
            }
        } catch (const std::exception& ex) {
          std::fprintf(stderr, "thread %d: %s\n", t, ex.what());
          ++errors;
        }
      });
    for (auto& th : ths) th.join();
    const double thr_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / rounds;
    db.check(ek_worker_batch_stats(db.handle(), &c2, &b2));
    // the reference's malformed-request cases must come back as errors, not crashes
    int rejected = 0;
    try { ek::ForwardReq bad = reqs[0]; bad.sequences.clear(); gate.forward(bad); } catch (const ek::EKError& e) { rejected += e.status() == EK_INVALID_INPUT; }
    try { ek::ForwardReq bad = reqs[0]; bad.sequences[0].experts[0] = ids[E - 1]; gate.forward(bad); } catch (const ek::EKError& e) { rejected += e.status() == EK_INVALID_INPUT; }
    try { db.load("shim/l0-e99999"); } catch (const ek::EKError& e) { rejected += e.status() == EK_EXPERT_NOT_FOUND; }
    db.remove(ids[0]);
    try { gate.forward(reqs[0]); } catch (const ek::EKError& e) { rejected += e.status() == EK_EXPERT_NOT_FOUND; }
    std::printf("{\"experts\": %d, \"rows\": %d, \"threads\": %d, \"rounds\": %d, \"one_thread_ms_per_round\": %.3f, "
                "\"threads_ms_per_round\": %.3f, \"one_thread_calls\": %lld, \"one_thread_passes\": %lld, "
                "\"threads_calls\": %lld, \"threads_passes\": %lld, \"mismatches\": %d, \"errors\": %d, \"rejected\": %d}\n",
                E, n, n_threads, rounds, seq_ms, thr_ms, (long long)(c1 - c0), (long long)(b1 - b0), (long long)(c2 - c1),
                (long long)(b2 - b1), mismatches.load(), errors.load(), rejected);
    return (mismatches.load() == 0 && errors.load() == 0 && rejected == 4) ? 0 : 2;
  } catch (const ek::EKError& e) {
    std::fprintf(stderr, "%s\n", e.what());
    return e.status() == EK_CUDA ? 3 : 2;
  }
}
