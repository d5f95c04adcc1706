// q35run: run roles of libq35b200.so from files, by tensor name -- the native host of the library, doing for it what
// the reference's board programs do for a compiled NPU kernel (tools/board/axrun.cc: inputs <dir>/<name>.bin, outputs
// out_<name>.bin, timed repetitions, outputs aliased onto inputs; tools/board/iojson.c: the IO table as JSON;
// tools/board/mc_stress.cc: repeated runs compared bit for bit with the first; tools/board/par_test.cc: N host threads
// running replicas at once; tools/board/mc_alt.cc: several kernels alternated like a layer chain, outputs poisoned).
//
//   q35run --roles                      names of all roles
//   q35run --io <role>                  the role's IO table as JSON (needs no GPU)
//   q35run <role> <dir> [reps] [--check R]
//       <dir>/io.txt lists the tensors of the call, one per line:  in|out <name> <dtype code> <d0> <d1> ...
//       (written by ax_dsl_kernels_b200.casefile.dump_case).  Inputs are read from <dir>/<name>.bin (missing: zeros),
//       a `workspace` of q35_workspace_bytes() is added when the role needs one, outputs go to <dir>/out_<name>.bin.
//       reps (default 20) further runs are timed with CUDA events.  --check R: R more runs from the same inputs,
//       every output compared bitwise with the first run's (a determinism / race check).
//       Q35RUN_ALIAS="state_out:state_in,...": that output lives in the input's buffer (in-place state, KV rows).
//   q35run --par N <role> <dir> [--rounds R]
//       N host threads, each with its own stream, its own copy of every buffer and its own workspace, call the role
//       together, with a barrier after every round: per-round time, the aggregate bandwidth of the inputs read, and
//       every replica's outputs compared bit for bit with replica 0's (the library is re-entrant per stream).
//   q35run --alt <role> <dir> [<role> <dir> ...] [--rounds R]
//       every round calls each case once, in order, on one stream.  From round 1 on the outputs are filled with 0xFF
//       bytes before the call and compared with round 0 after it: a role that leaves part of an output unwritten, or
//       depends on what its outputs held, shows up as a mismatch.
// Exit status: 0 ok, 1 run or comparison failed, 2 usage.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "q35b200.h"

namespace {

struct Entry {
  bool is_out = false;
  std::string name;
  int dtype = 0;
  std::vector<int64_t> shape;
  size_t bytes = 0;
  void* dev = nullptr;
  int alias_of = -1;  // output sharing an input's buffer
};

size_t elem_bits(int dtype) {
  switch (dtype) {
    case Q35_U8: case Q35_E4M3: return 8;
    case Q35_F32: case Q35_I32: return 32;
    case Q35_BF16: case Q35_F16: return 16;
    case Q35_FP4: return 4;
    default: return 0;
  }
}

bool read_file(const std::string& path, std::vector<char>* out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  out->assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
  return true;
}

int fail(const char* what) {
  fprintf(stderr, "q35run: %s: %s\n", what, q35_last_error());
  return 1;
}

#define CUDA_OK(call)                                                                  \
  do {                                                                                 \
    cudaError_t e_ = (call);                                                           \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "q35run: %s: %s\n", #call, cudaGetErrorString(e_));              \
      return 1;                                                                        \
    }                                                                                  \
  } while (0)

// One call of one role with its own device buffers: the tensors of <dir>/io.txt, inputs from <dir>/<name>.bin.
struct Case {
  std::string role, dir;
  std::vector<Entry> io;
  std::vector<std::vector<char>> host_in;
  std::vector<q35_io> call;
  size_t in_bytes = 0;

  int parse(bool verbose) {
    std::ifstream f(dir + "/io.txt");
    if (!f) { fprintf(stderr, "q35run: cannot open %s/io.txt\n", dir.c_str()); return 2; }
    std::string line;
    while (std::getline(f, line)) {
      std::istringstream ls(line);
      std::string kind;
      Entry e;
      if (!(ls >> kind >> e.name >> e.dtype)) continue;
      e.is_out = kind == "out";
      int64_t d, n = 1;
      while (ls >> d) { e.shape.push_back(d); n *= d; }
      if (e.shape.size() > 6 || !elem_bits(e.dtype)) { fprintf(stderr, "q35run: bad line: %s\n", line.c_str()); return 2; }
      e.bytes = size_t(n) * elem_bits(e.dtype) / 8;
      io.push_back(e);
    }
    if (const char* alias = getenv("Q35RUN_ALIAS")) {
      std::istringstream as(alias);
      std::string pair;
      while (std::getline(as, pair, ',')) {
        const size_t c = pair.find(':');
        if (c == std::string::npos) continue;
        const std::string on = pair.substr(0, c), in = pair.substr(c + 1);
        for (size_t o = 0; o < io.size(); ++o)
          for (size_t i = 0; i < io.size(); ++i)
            if (io[o].is_out && io[o].name == on && !io[i].is_out && io[i].name == in && io[i].bytes == io[o].bytes)
              io[o].alias_of = int(i);
      }
    }
    host_in.resize(io.size());
    for (size_t i = 0; i < io.size(); ++i) {
      Entry& e = io[i];
      if (e.is_out) continue;
      const bool found = read_file(dir + "/" + e.name + ".bin", &host_in[i]);
      if (found && host_in[i].size() != e.bytes) {
        fprintf(stderr, "q35run: %s.bin has %zu bytes, the table says %zu\n", e.name.c_str(), host_in[i].size(), e.bytes);
        return 1;
      }
      if (!found) host_in[i].assign(e.bytes, 0);
      in_bytes += e.bytes;
      if (verbose) printf("in  %-16s %12zu bytes%s\n", e.name.c_str(), e.bytes, found ? "" : " (zeros)");
    }
    return 0;
  }

  void bind() {
    call.clear();
    for (const Entry& e : io) {
      q35_io b{};
      b.name = e.name.c_str(); b.ptr = e.dev; b.bytes = e.bytes; b.dtype = e.dtype; b.ndim = int(e.shape.size());
      for (size_t d = 0; d < e.shape.size(); ++d) b.shape[d] = e.shape[d];
      call.push_back(b);
    }
  }

  int allocate(bool verbose) {
    for (Entry& e : io) {
      if (e.alias_of >= 0) continue;
      CUDA_OK(cudaMalloc(&e.dev, e.bytes ? e.bytes : 16));
      CUDA_OK(cudaMemset(e.dev, 0, e.bytes ? e.bytes : 16));
    }
    for (Entry& e : io)
      if (e.alias_of >= 0) {
        e.dev = io[size_t(e.alias_of)].dev;
        if (verbose) printf("out %-16s in place of input %s\n", e.name.c_str(), io[size_t(e.alias_of)].name.c_str());
      }
    bind();
    const int64_t ws_bytes = q35_workspace_bytes(role.c_str(), call.data(), int(call.size()));
    if (ws_bytes < 0) return fail("workspace size");
    if (ws_bytes > 0) {
      Entry w;
      w.name = "workspace"; w.dtype = Q35_U8; w.shape = {ws_bytes}; w.bytes = size_t(ws_bytes);
      w.is_out = true;  // nothing to upload; not written to a file either
      CUDA_OK(cudaMalloc(&w.dev, w.bytes));
      io.push_back(w);
      host_in.emplace_back();
      bind();
      if (verbose) printf("in  %-16s %12lld bytes (scratch)\n", "workspace", (long long)ws_bytes);
    }
    return 0;
  }

  int upload(cudaStream_t s) {
    for (size_t i = 0; i < io.size(); ++i)
      if (!io[i].is_out) CUDA_OK(cudaMemcpyAsync(io[i].dev, host_in[i].data(), io[i].bytes, cudaMemcpyHostToDevice, s));
    CUDA_OK(cudaStreamSynchronize(s));
    return 0;
  }

  bool real_output(size_t i) const { return io[i].is_out && io[i].name != "workspace"; }

  int poison_outputs(cudaStream_t s) {
    for (size_t i = 0; i < io.size(); ++i)
      if (real_output(i) && io[i].alias_of < 0) CUDA_OK(cudaMemsetAsync(io[i].dev, 0xFF, io[i].bytes, s));
    return 0;
  }

  int run(cudaStream_t s) { return q35_run(role.c_str(), call.data(), int(call.size()), s); }

  int download(std::vector<std::vector<char>>* out, cudaStream_t s) {
    out->assign(io.size(), {});
    for (size_t i = 0; i < io.size(); ++i) {
      if (!real_output(i)) continue;
      (*out)[i].resize(io[i].bytes);
      CUDA_OK(cudaMemcpyAsync((*out)[i].data(), io[i].dev, io[i].bytes, cudaMemcpyDeviceToHost, s));
    }
    CUDA_OK(cudaStreamSynchronize(s));
    return 0;
  }
};

// reusable barrier for the replica threads
class Barrier {
 public:
  explicit Barrier(int n) : n_(n) {}
  void wait() {
    std::unique_lock<std::mutex> lk(m_);
    const int gen = gen_;
    if (++count_ == n_) { count_ = 0; ++gen_; cv_.notify_all(); }
    else cv_.wait(lk, [&] { return gen_ != gen; });
  }
 private:
  std::mutex m_;
  std::condition_variable cv_;
  int n_, count_ = 0, gen_ = 0;
};

int mode_par(int n, const std::string& role, const std::string& dir, int rounds) {
  std::vector<Case> reps(static_cast<size_t>(n));
  for (int i = 0; i < n; ++i) {
    reps[size_t(i)].role = role; reps[size_t(i)].dir = dir;
    if (int rc = reps[size_t(i)].parse(i == 0)) return rc;
    if (int rc = reps[size_t(i)].allocate(i == 0)) return rc;
  }
  Barrier bar(n + 1);
  std::vector<std::vector<std::vector<char>>> outs(static_cast<size_t>(n));
  std::atomic<int> failures{0};
  std::vector<std::thread> th;
  for (int i = 0; i < n; ++i) {
    th.emplace_back([&, i] {
      Case& c = reps[size_t(i)];
      cudaStream_t s;
      if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { ++failures; }
      if (c.upload(s)) ++failures;
      bar.wait();  // everybody loaded
      for (int r = 0; r < rounds; ++r) {
        if (c.run(s)) { if (failures++ < 3) fprintf(stderr, "q35run: replica %d round %d: %s\n", i, r, q35_last_error()); }
        if (cudaStreamSynchronize(s) != cudaSuccess) ++failures;
        bar.wait();  // the per-round meeting point a tensor-parallel split would need
      }
      if (c.download(&outs[size_t(i)], s)) ++failures;
      cudaStreamDestroy(s);
    });
  }
  bar.wait();
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < rounds; ++r) bar.wait();
  const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / rounds;
  for (auto& t : th) t.join();
  int differing = 0;
  const bool in_place = getenv("Q35RUN_ALIAS") != nullptr;  // in-place state evolves identically on every replica
  for (int i = 1; i < n; ++i)
    for (size_t k = 0; k < outs[0].size(); ++k)
      if (!outs[0][k].empty() && outs[size_t(i)][k] != outs[0][k]) {
        ++differing;
        printf("replica %d: output %s differs from replica 0\n", i, reps[0].io[k].name.c_str());
      }
  (void)in_place;
  printf("RESULT par=%d rounds=%d us_per_round=%.1f input_GBps=%.1f differing=%d run_failures=%d device_status=%d\n", n,
         rounds, us, double(reps[0].in_bytes) * n / us / 1e3, differing, failures.load(), q35_device_status(nullptr));
  return (differing || failures.load()) ? 1 : 0;
}

int mode_alt(const std::vector<std::pair<std::string, std::string>>& pairs, int rounds) {
  std::vector<Case> cs(pairs.size());
  for (size_t i = 0; i < pairs.size(); ++i) {
    cs[i].role = pairs[i].first; cs[i].dir = pairs[i].second;
    if (int rc = cs[i].parse(false)) return rc;
    if (int rc = cs[i].allocate(false)) return rc;
    if (cs[i].upload(nullptr)) return 1;
  }
  std::vector<std::vector<std::vector<char>>> ref(cs.size());
  std::vector<int> fails(cs.size(), 0), mism(cs.size(), 0);
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < rounds; ++r)
    for (size_t i = 0; i < cs.size(); ++i) {
      Case& c = cs[i];
      if (r > 0 && c.poison_outputs(nullptr)) return 1;
      if (c.upload(nullptr)) return 1;  // in-place outputs restart from the same inputs every round
      if (c.run(nullptr)) {
        if (fails[i]++ < 3) printf("round %d %s: %s\n", r, c.role.c_str(), q35_last_error());
        continue;
      }
      std::vector<std::vector<char>> now;
      if (c.download(&now, nullptr)) return 1;
      if (r == 0) { ref[i] = now; continue; }
      for (size_t k = 0; k < now.size(); ++k)
        if (!now[k].empty() && now[k] != ref[i][k] && mism[i]++ < 3) {
          size_t off = 0;
          while (off < now[k].size() && now[k][off] == ref[i][k][off]) ++off;
          printf("round %d %s: output %s differs from round 0 (first byte %zu of %zu)\n", r, c.role.c_str(),
                 c.io[k].name.c_str(), off, now[k].size());
        }
    }
  const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / rounds;
  int bad = 0;
  for (size_t i = 0; i < cs.size(); ++i) {
    printf("RESULT %s %s fails=%d mismatches=%d\n", cs[i].role.c_str(), cs[i].dir.c_str(), fails[i], mism[i]);
    bad += fails[i] + mism[i];
  }
  const int status = q35_device_status(nullptr);
  printf("RESULT rounds=%d ms_per_round=%.3f device_status=%d\n", rounds, ms, status);
  return (bad || status) ? 1 : 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc >= 2 && !strcmp(argv[1], "--roles")) {
    for (int i = 0; i < q35_role_count(); ++i) printf("%s\n", q35_role_name(i));
    return 0;
  }
  if (argc >= 3 && !strcmp(argv[1], "--io")) {
    const int need = q35_io_table(argv[2], nullptr, 0);
    if (need < 0) return fail("io table");
    std::vector<char> buf(size_t(need) + 1);
    q35_io_table(argv[2], buf.data(), buf.size());
    printf("%s\n", buf.data());
    return 0;
  }
  if (argc >= 5 && !strcmp(argv[1], "--par")) {
    const int n = atoi(argv[2]);
    int rounds = 20;
    for (int i = 5; i + 1 < argc; ++i)
      if (!strcmp(argv[i], "--rounds")) rounds = atoi(argv[i + 1]);
    if (n < 1 || n > 64 || rounds < 1) { fprintf(stderr, "q35run: --par N (1..64) <role> <dir> [--rounds R]\n"); return 2; }
    return mode_par(n, argv[3], argv[4], rounds);
  }
  if (argc >= 4 && !strcmp(argv[1], "--alt")) {
    std::vector<std::pair<std::string, std::string>> pairs;
    int rounds = 10, i = 2;
    for (; i + 1 < argc && strcmp(argv[i], "--rounds"); i += 2) pairs.emplace_back(argv[i], argv[i + 1]);
    if (i + 1 < argc && !strcmp(argv[i], "--rounds")) rounds = atoi(argv[i + 1]);
    if (pairs.empty() || rounds < 2) { fprintf(stderr, "q35run: --alt <role> <dir> [...] [--rounds R >= 2]\n"); return 2; }
    return mode_alt(pairs, rounds);
  }
  if (argc < 3) {
    fprintf(stderr, "usage: q35run --roles | --io <role> | <role> <dir> [reps] [--check R] | --par N <role> <dir> "
                    "[--rounds R] | --alt <role> <dir> [...] [--rounds R]\n");
    return 2;
  }
  Case c;
  c.role = argv[1]; c.dir = argv[2];
  int reps = 20, check = 0;
  for (int i = 3; i < argc; ++i) {
    if (!strcmp(argv[i], "--check") && i + 1 < argc) check = atoi(argv[++i]);
    else reps = atoi(argv[i]);
  }
  if (int rc = c.parse(true)) return rc;
  if (int rc = c.allocate(true)) return rc;

  // ---- first run, outputs to files
  if (c.upload(nullptr)) return 1;
  if (c.run(nullptr)) return fail("run");
  std::vector<std::vector<char>> first;
  if (c.download(&first, nullptr)) return 1;
  for (size_t i = 0; i < c.io.size(); ++i) {
    if (first[i].empty() && !(c.real_output(i) && c.io[i].bytes == 0)) continue;
    const Entry& e = c.io[i];
    const std::string path = c.dir + "/out_" + e.name + ".bin";
    std::ofstream(path, std::ios::binary).write(first[i].data(), std::streamsize(e.bytes));
    printf("out %-16s %12zu bytes -> %s\n", e.name.c_str(), e.bytes, path.c_str());
  }

  // ---- repeated runs from the same inputs must reproduce the first bit for bit
  int bad = 0;
  for (int r = 0; r < check; ++r) {
    if (c.upload(nullptr)) return 1;
    if (c.run(nullptr)) return fail("run (check)");
    std::vector<std::vector<char>> now;
    if (c.download(&now, nullptr)) return 1;
    for (size_t i = 0; i < now.size(); ++i)
      if (!first[i].empty() && now[i] != first[i]) {
        ++bad;
        printf("check run %d: output %s differs from the first run\n", r, c.io[i].name.c_str());
      }
  }
  if (check) printf("check: %d runs, %d differing outputs\n", check, bad);

  // ---- timing (in-place outputs keep evolving, as a recurrent state does)
  if (reps > 0) {
    cudaEvent_t t0, t1;
    CUDA_OK(cudaEventCreate(&t0));
    CUDA_OK(cudaEventCreate(&t1));
    CUDA_OK(cudaEventRecord(t0));
    for (int r = 0; r < reps; ++r)
      if (c.run(nullptr)) return fail("run (timed)");
    CUDA_OK(cudaEventRecord(t1));
    CUDA_OK(cudaEventSynchronize(t1));
    float ms = 0.f;
    CUDA_OK(cudaEventElapsedTime(&ms, t0, t1));
    printf("%s: %.1f us per run over %d runs\n", c.role.c_str(), ms * 1e3f / float(reps), reps);
  }
  const int status = q35_device_status(nullptr);
  printf("device status %d\n", status);
  return (bad || status) ? 1 : 0;
}
