// Stress test of the copy engine's host-side logic on the CPU: the real
// offload_engine.cpp is compiled against the stand-in runtime in fake_cuda/ (streams are
// threads with random delays and bounded queues) and a stand-in "kernel" that adds
// known constants to every element it is given.  After S steps every element of the
// host state must hold its initial value plus S times the constants: a chunk that was
// stepped twice or not at all, loaded before its previous write-back had finished,
// overwritten in the staging buffer before it was written back, or mixed up with
// another tensor shows up as a wrong value.  Built with -fsanitize=thread the same run
// checks the helper threads' use of the engine's data structures.
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <vector>

#include "../../offload_adam_b200/csrc/offload_engine.cpp"

namespace oab {
// stand-in kernel: m += 1, v += 2, extra(fp32) += 3 + g, p = m
cudaError_t launch_adam_step(const AdamStepArgs& a, cudaStream_t s) {
  AdamStepArgs c = a;
  s->push([c] {
    uint16_t* m = static_cast<uint16_t*>(c.m);
    uint16_t* v = static_cast<uint16_t*>(c.v);
    float* x = static_cast<float*>(c.extra);
    const uint16_t* g = static_cast<const uint16_t*>(c.g);
    uint16_t* p = static_cast<uint16_t*>(c.p);
    for (int64_t i = 0; i < c.n; ++i) {
      m[i] = (uint16_t)(m[i] + 1);
      v[i] = (uint16_t)(v[i] + 2);
      if (x) x[i] += 3.0f + (g ? (float)g[i] : 0.0f);
      if (p) p[i] = m[i];
    }
    // deliberate overrun (canary scenario): the first word behind the chunk's last sub-buffer
    if (c.max_ctas == -7 && x) x[((4 * c.n + 255) / 256 * 256) / 4] = 1.0f;
  });
  return cudaSuccess;
}
// stand-in for the step of a quantized weight: the same update, plus one "packed" byte
// per element (the low byte of the new m) stored at the element's place in the whole
// weight, which checks the row arithmetic of chunked launches
cudaError_t launch_adam_quant_push(const AdamStepArgs& a, const QuantPushArgs& q, cudaStream_t s) {
  if (a.n % q.in_f != 0) return cudaErrorInvalidValue;
  launch_adam_step(a, s);
  AdamStepArgs c = a;
  QuantPushArgs qq = q;
  s->push([c, qq] {
    const uint16_t* m = static_cast<const uint16_t*>(c.m);
    for (int r = 0; r < qq.n_replicas; ++r) {
      uint8_t* out = static_cast<uint8_t*>(qq.payload0[r]) + qq.row0 * qq.in_f;
      for (int64_t i = 0; i < c.n; ++i) out[i] = (uint8_t)m[i];
    }
  });
  return cudaSuccess;
}
// stand-in for the guard check (the real one is a kernel in grad_ops.cu)
cudaError_t launch_check_canary(const void* guard, int words, int* status, int tag, cudaStream_t s) {
  s->push([=] {
    const uint32_t* g = static_cast<const uint32_t*>(guard);
    for (int i = 0; i < words; ++i)
      if (g[i] != kCanaryWord && status[0] == 0) { status[0] = 1; status[1] = tag; }
  });
  return cudaSuccess;
}
// when set, the stand-in step kernel of this tensor writes one element past its moments
static std::atomic<int> g_overrun_pid{-1};
// stand-in accumulate: out = a + b (uint16 arithmetic)
cudaError_t launch_grad_accumulate(const AccumArgs& a, cudaStream_t s) {
  AccumArgs c = a;
  s->push([c] {
    uint16_t* out = static_cast<uint16_t*>(c.out);
    const uint16_t* x = static_cast<const uint16_t*>(c.a);
    const uint16_t* y = static_cast<const uint16_t*>(c.b);
    for (int64_t i = 0; i < c.n; ++i) out[i] = (uint16_t)(x[i] + (y ? y[i] : 0));
  });
  return cudaSuccess;
}
}  // namespace oab

using oab::OffloadEngine;

struct Tensor {
  int64_t n;
  int stepped = 0;  // how many steps this tensor has taken
  std::vector<uint16_t> m, v, p, g, hg;  // m, v: host state; p, g: "device"; hg: host gradient
  std::vector<float> x;
  std::vector<uint16_t> m0, v0;
  std::vector<float> x0;
  std::vector<uint8_t> packed;  // "payload" of a quantized weight (stand-in)
};
constexpr int64_t kInF = 8;  // row length of the stand-in quantized weights

static uint16_t seed_val(int pid, int64_t i, int salt) { return (uint16_t)((pid * 131 + i * 7 + salt * 1009) & 0x3fff); }

struct Scenario {
  const char* name;
  int tensors, steps;
  int64_t chunk;
  double ring_fraction;  // staging buffer as a fraction of the whole state (<= 0: the minimum)
  bool async_writeback, thread_prefetch, call_prefetch, shuffle_order;
  size_t queue_capacity;
  bool host_grads = false;  // gradients live on the host and are loaded with the state
  bool destroy_busy = false;  // destroy the engine with transfers in flight: its destructor must finish them
  bool chaos = false;  // skipped tensors, repeated and cancelled plans, discards between steps
  int slow_h2d_us = 0, slow_d2h_us = 0;  // extra time per operation of the copy streams
  int resident = 0;    // this many tensors (the last ones) keep their state in the staging buffer
  bool canaries = false;  // guard words behind every chunk and resident tensor
  bool overrun = false;   // the stand-in kernel writes past its operands: synchronize() must say so
  bool quant = false;  // tensors are whole rows of kInF elements, stepped through the quantizing launch
                       // in chunks of their own size
  bool lazy = false;   // resident state goes back to the host only at wait_writebacks()/synchronize()
};

static int run(const Scenario& sc, unsigned seed) {
  fake_cuda::queue_capacity = sc.queue_capacity;
  std::mt19937 rng(seed);
  std::vector<Tensor> ts(sc.tensors);
  size_t state_bytes = 0;
  for (int t = 0; t < sc.tensors; ++t) {
    Tensor& T = ts[t];
    T.n = 1 + rng() % (5 * sc.chunk);  // ragged: several chunks and a tail
    if (sc.quant) T.n = (T.n + kInF - 1) / kInF * kInF;
    T.packed.assign(T.n, 0);
    T.m.resize(T.n); T.v.resize(T.n); T.x.resize(T.n); T.p.assign(T.n, 0); T.g.resize(T.n); T.hg.assign(T.n, 0);
    for (int64_t i = 0; i < T.n; ++i) {
      T.m[i] = seed_val(t, i, 1); T.v[i] = seed_val(t, i, 2); T.x[i] = (float)seed_val(t, i, 3);
      T.g[i] = (uint16_t)((t * 7 + i) % 5);
    }
    T.m0 = T.m; T.v0 = T.v; T.x0 = T.x;
    state_bytes += T.n * 8;
  }
  fake_cuda::Stream compute(seed + 1), h2d(seed + 2), d2h(seed + 3);
  h2d.extra_delay_us = sc.slow_h2d_us;
  d2h.extra_delay_us = sc.slow_d2h_us;
  oab::EngineOptions opt;
  opt.chunk_elems = sc.chunk;
  opt.async_writeback = sc.async_writeback;
  opt.canaries = sc.canaries;
  opt.lazy_resident = sc.lazy;
  if (sc.overrun) opt.max_ctas = -7;
  bool caught = false;
  size_t ring = OffloadEngine::min_ring_bytes(sc.chunk);
  if (sc.ring_fraction > 0) ring = std::max(ring, (size_t)(state_bytes * sc.ring_fraction) / 256 * 256);
  size_t resident_need = 0;
  for (int t = sc.tensors - sc.resident; t < sc.tensors; ++t)
    resident_need += 2 * ((2 * ts[t].n + 255) / 256 * 256) + (4 * ts[t].n + 255) / 256 * 256;
  ring += resident_need + (sc.canaries ? 256 * (size_t)(sc.resident + 8) : 0);
  void* ws = aligned_alloc(256, ring);
  int bad = 0;
  try {
  // per-tensor chunk of the quantized stand-ins: whole rows, not the engine's default
  const int64_t qchunk = sc.quant ? std::max<int64_t>(kInF, (sc.chunk - 3) / kInF * kInF) : 0;
  {
    OffloadEngine eng(0, &compute, &h2d, &d2h, ws, ring, opt, sc.tensors);
    for (int t = sc.tensors - sc.resident; t < sc.tensors; ++t)
      if (!eng.make_resident(t, oab::kModeFP32Master, ts[t].n)) { fprintf(stderr, "%s: make_resident refused\n", sc.name); ++bad; }
    std::vector<int> order(sc.tensors);
    for (int t = 0; t < sc.tensors; ++t) order[t] = t;
    for (int step = 0; step < sc.steps; ++step) {
      // "forward/backward": time for the early loads of this step
      std::this_thread::sleep_for(std::chrono::microseconds(rng() % 3000));
      if (sc.call_prefetch) {  // loads issued from the training thread, a few chunks at a time
        for (int t = 0; t < sc.tensors; ++t) {
          oab::StagedStepArgs a;
          a.pid = t; a.k.mode = oab::kModeFP32Master; a.k.n = ts[t].n;
          a.k.m = ts[t].m.data(); a.k.v = ts[t].v.data(); a.k.extra = ts[t].x.data();
          a.chunk = qchunk;
          bool full = false;
          int64_t off = 0;
          while (off < ts[t].n && !full) {
            int64_t now = eng.prefetch(a, off, 1 + rng() % 2, 1 + rng() % 2, &full);
            if (now == off) std::this_thread::sleep_for(std::chrono::microseconds(50));
            off = now;
          }
          if (full) break;
        }
      }
      std::vector<int> step_order = order;
      if (sc.shuffle_order && step % 2 == 1) std::shuffle(step_order.begin(), step_order.end(), rng);
      if (sc.host_grads)  // what the gradient hooks of the last micro-batch do
        for (int t = 0; t < sc.tensors; ++t)
          eng.staged_grad_to_host(t, ts[t].hg.data(), ts[t].g.data(), ts[t].n, /*first=*/true, nullptr, nullptr);
      for (int t : step_order) {
        Tensor& T = ts[t];
        if (sc.chaos && rng() % 5 == 0) continue;  // no gradient for this tensor in this step
        ++T.stepped;
        oab::StagedStepArgs a;
        a.pid = t;
        a.k.mode = oab::kModeFP32Master;
        a.k.n = T.n;
        a.k.p = T.p.data();
        if (sc.host_grads) a.host_grad = T.hg.data();
        else a.k.g = T.g.data();
        a.k.m = T.m.data(); a.k.v = T.v.data(); a.k.extra = T.x.data();
        oab::QuantPushArgs q;
        if (sc.quant) {
          q.format = oab::kQInt8; q.in_f = kInF; q.out_f = T.n / kInF; q.row0 = 0; q.n_replicas = 1;
          q.payload0[0] = T.packed.data(); q.payload1[0] = T.packed.data();
          a.quant = &q;
          a.chunk = qchunk;
        }
        eng.staged_step(a);
      }
      eng.join_compute(&compute);
      if (rng() % 4 == 0) eng.wait_writebacks();
      if (rng() % 7 == 0) eng.synchronize();
      if (rng() % 9 == 0) eng.join(&compute);
      if (sc.thread_prefetch) {  // plan for the next step, as the optimizer hands it over
        std::vector<OffloadEngine::PrefetchItem> plan;
        for (int t : order) {
          OffloadEngine::PrefetchItem it;
          it.pid = t; it.mode = oab::kModeFP32Master; it.n = ts[t].n;
          it.m = ts[t].m.data(); it.v = ts[t].v.data(); it.extra = ts[t].x.data();
          it.chunk = qchunk;
          plan.push_back(it);
        }
        eng.start_prefetch(plan, 1 + rng() % 3);
        if (sc.chaos) {
          switch (rng() % 5) {
            case 0: eng.stop_prefetch(); break;
            case 1: eng.discard_prefetched(); break;
            case 2: eng.start_prefetch(plan, 2); break;  // a second plan replaces the first
            case 3: std::this_thread::sleep_for(std::chrono::microseconds(300)); eng.discard_prefetched();
                    eng.start_prefetch(plan, 1); break;
            default: break;
          }
        }
      }
    }
    // gradient round trip through the buffer, mixed with whatever is still in flight
    for (int t = 0; t < sc.tensors; ++t) {
      eng.staged_grad_to_host(t, ts[t].hg.data(), ts[t].g.data(), ts[t].n, /*first=*/true, nullptr, nullptr);
      eng.staged_grad_to_host(t, ts[t].hg.data(), ts[t].g.data(), ts[t].n, /*first=*/false, nullptr, nullptr);
    }
    if (!sc.destroy_busy) eng.synchronize();
  }
  } catch (const std::runtime_error& e) {
    if (sc.overrun && std::string(e.what()).find("guard") != std::string::npos) caught = true;
    else { fprintf(stderr, "%s: unexpected error: %s\n", sc.name, e.what()); ++bad; }
  }
  if (sc.overrun) {
    if (!caught) { fprintf(stderr, "%s: the overrun was not reported\n", sc.name); ++bad; }
    free(ws);
    printf("%-28s seed %u: %s\n", sc.name, seed, bad ? "FAILED" : "ok (overrun reported)");
    return bad;
  }
  for (int t = 0; t < sc.tensors; ++t) {
    const Tensor& T = ts[t];
    for (int64_t i = 0; i < T.n; ++i) {
      const uint16_t wm = (uint16_t)(T.m0[i] + T.stepped), wv = (uint16_t)(T.v0[i] + 2 * T.stepped);
      const float wx = T.x0[i] + (3.0f + (float)T.g[i]) * T.stepped;
      if (T.stepped == 0 && T.p[i] == 0) continue;  // never stepped: p was never written
      const bool packed_ok = !sc.quant || T.packed[i] == (uint8_t)wm;
      if (T.m[i] != wm || T.v[i] != wv || T.x[i] != wx || T.p[i] != wm || T.hg[i] != (uint16_t)(2 * T.g[i]) || !packed_ok) {
        // (the final gradient round trip leaves hg = g + g in every scenario)
        if (bad < 5)
          fprintf(stderr, "%s: tensor %d elem %lld: m %u/%u v %u/%u x %g/%g p %u hg %u/%u\n", sc.name, t,
                  (long long)i, T.m[i], wm, T.v[i], wv, T.x[i], wx, T.p[i], T.hg[i], 2 * T.g[i]);
        ++bad;
      }
    }
  }
  free(ws);
  printf("%-28s seed %u: %s (%ld stream operations)\n", sc.name, seed, bad ? "FAILED" : "ok",
         fake_cuda::ops_executed.load());
  return bad;
}

int main(int argc, char** argv) {
  const int rounds = argc > 1 ? atoi(argv[1]) : 3;
  const Scenario scenarios[] = {
      //  name                     tensors steps chunk ring  async thread call  shuffle capacity
      {"large ring, inline",            6, 4,   64, 2.0,  false, false, false, false, 64},
      {"minimal ring, inline",          6, 4,   64, 0.0,  false, false, false, false, 64},
      {"minimal ring, writer thread",   6, 5,   64, 0.0,  true,  false, false, false, 16},
      {"half ring, both threads",       9, 6,   64, 0.5,  true,  true,  false, false, 16},
      {"full ring, both threads",       9, 6,   64, 1.1,  true,  true,  false, false, 24},
      {"small ring, both threads",      9, 6,   32, 0.15, true,  true,  false, false, 8},
      {"loads from training thread",    7, 5,   64, 0.6,  true,  false, true,  false, 32},
      {"out-of-order steps",            7, 6,   64, 0.7,  true,  true,  false, true,  32},
      {"host gradients",                6, 5,   64, 0.3,  true,  true,  false, false, 16, true},
      {"many chunks, tiny queues",     12, 8,   16, 0.4,  true,  true,  false, false, 6},
      {"destroyed while busy",          8, 4,   64, 0.5,  true,  true,  false, false, 16, false, true},
      {"chaos",                         9, 10,  32, 0.6,  true,  true,  false, true,  12, false, false, true},
      {"slow write-backs",              8, 5,   64, 1.1,  true,  true,  false, false, 12, false, false, false, 0, 150},
      {"slow loads",                    8, 5,   64, 0.4,  true,  true,  false, false, 12, false, false, false, 150, 0},
      //                                                                                      hostg  busy   chaos  slow    resident quant
      {"all resident",                  6, 6,   64, 0.0,  true,  true,  false, false, 16, false, false, false, 0, 0,   6},
      {"half resident, small ring",     9, 6,   32, 0.15, true,  true,  false, false, 8,  false, false, false, 0, 0,   4},
      {"resident, inline, no plans",    6, 5,   64, 0.0,  false, false, false, false, 64, false, false, false, 0, 0,   3},
      {"resident, chaos",               9, 10,  32, 0.5,  true,  true,  false, true,  12, false, false, true,  0, 0,   5},
      {"resident, slow write-backs",    8, 5,   64, 0.3,  true,  true,  false, false, 12, false, false, false, 0, 150, 4},
      {"resident, destroyed busy",      8, 4,   64, 0.3,  true,  true,  false, false, 16, false, true,  false, 0, 0,   4},
      {"row chunks, quantizing launch", 8, 5,   64, 0.4,  true,  true,  false, false, 16, false, false, false, 0, 0,   0, false, false, true},
      {"row chunks, resident",          8, 5,   64, 0.4,  true,  true,  false, true,  16, false, false, false, 0, 0,   3, false, false, true},
      {"row chunks, caller loads",      7, 5,   64, 0.6,  true,  false, true,  false, 32, false, false, false, 0, 0,   0, false, false, true},
      //                                                                                                                    resident canaries overrun quant
      {"canaries, ring",                8, 5,   64, 0.4,  true,  true,  false, false, 16, false, false, false, 0, 0,   0, true},
      {"canaries, resident + ring",     8, 5,   64, 0.3,  true,  true,  false, true,  16, false, false, false, 0, 0,   4, true},
      {"canaries, host gradients",      6, 5,   64, 0.3,  true,  true,  false, false, 16, true,  false, false, 0, 0,   0, true},
      {"canaries report an overrun",    6, 3,   64, 0.5,  false, false, false, false, 64, false, false, false, 0, 0,   0, true, true},
      {"canaries, resident overrun",    6, 3,   64, 0.5,  true,  true,  false, false, 16, false, false, false, 0, 0,   6, true, true},
      //                                                                                                                    resident canaries overrun quant lazy
      {"lazy resident, all",            6, 8,   64, 0.0,  true,  true,  false, false, 16, false, false, false, 0, 0,   6, false, false, false, true},
      {"lazy resident + ring",          9, 8,   32, 0.15, true,  true,  false, true,  8,  false, false, false, 0, 0,   4, false, false, false, true},
      {"lazy resident, inline",         6, 6,   64, 0.0,  false, false, false, false, 64, false, false, false, 0, 0,   3, false, false, false, true},
      {"lazy resident, chaos",          9, 10,  32, 0.5,  true,  true,  false, true,  12, false, false, true,  0, 0,   5, false, false, false, true},
      {"lazy resident, quantized",      8, 6,   64, 0.4,  true,  true,  false, true,  16, false, false, false, 0, 0,   3, true,  false, true,  true},
  };
  int bad = 0;
  for (int r = 0; r < rounds; ++r)
    for (const Scenario& sc : scenarios) bad += run(sc, 1000u * r + 17u);
  printf(bad ? "FAILED\n" : "all scenarios ok\n");
  return bad ? 1 : 0;
}
