// q35run: run one role of libq35b200.so from files, by tensor name -- the native host of the library, doing for it
// what the reference's board programs do for a compiled NPU kernel (tools/board/axrun.cc: inputs <dir>/<name>.bin,
// outputs out_<name>.bin, timed repetitions, outputs aliased onto inputs; tools/board/iojson.c: the IO table as JSON;
// tools/board/mc_stress.cc: repeated runs compared bit for bit with the first).
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
// Exit status: 0 ok, 1 run or comparison failed, 2 usage.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
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
  if (argc < 3) {
    fprintf(stderr, "usage: q35run --roles | --io <role> | <role> <dir> [reps] [--check R]\n");
    return 2;
  }
  const std::string role = argv[1], dir = argv[2];
  int reps = 20, check = 0;
  for (int i = 3; i < argc; ++i) {
    if (!strcmp(argv[i], "--check") && i + 1 < argc) check = atoi(argv[++i]);
    else reps = atoi(argv[i]);
  }

  // ---- the call's tensors
  std::vector<Entry> io;
  {
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

  // ---- device buffers
  std::vector<std::vector<char>> host_in(io.size());
  for (size_t i = 0; i < io.size(); ++i) {
    Entry& e = io[i];
    if (e.alias_of >= 0) continue;
    CUDA_OK(cudaMalloc(&e.dev, e.bytes ? e.bytes : 16));
    CUDA_OK(cudaMemset(e.dev, 0, e.bytes ? e.bytes : 16));
    if (!e.is_out) {
      const bool found = read_file(dir + "/" + e.name + ".bin", &host_in[i]);
      if (found && host_in[i].size() != e.bytes) {
        fprintf(stderr, "q35run: %s.bin has %zu bytes, the table says %zu\n", e.name.c_str(), host_in[i].size(), e.bytes);
        return 1;
      }
      if (!found) host_in[i].assign(e.bytes, 0);
      printf("in  %-16s %12zu bytes%s\n", e.name.c_str(), e.bytes, found ? "" : " (zeros)");
    }
  }
  for (Entry& e : io)
    if (e.alias_of >= 0) {
      e.dev = io[size_t(e.alias_of)].dev;
      printf("out %-16s in place of input %s\n", e.name.c_str(), io[size_t(e.alias_of)].name.c_str());
    }
  auto upload = [&]() -> int {
    for (size_t i = 0; i < io.size(); ++i)
      if (!io[i].is_out) CUDA_OK(cudaMemcpy(io[i].dev, host_in[i].data(), io[i].bytes, cudaMemcpyHostToDevice));
    return 0;
  };

  std::vector<q35_io> call;
  auto bind = [&]() {
    call.clear();
    for (const Entry& e : io) {
      q35_io b{};
      b.name = e.name.c_str(); b.ptr = e.dev; b.bytes = e.bytes; b.dtype = e.dtype; b.ndim = int(e.shape.size());
      for (size_t d = 0; d < e.shape.size(); ++d) b.shape[d] = e.shape[d];
      call.push_back(b);
    }
  };
  bind();
  const int64_t ws_bytes = q35_workspace_bytes(role.c_str(), call.data(), int(call.size()));
  if (ws_bytes < 0) return fail("workspace size");
  if (ws_bytes > 0) {
    Entry w;
    w.name = "workspace"; w.dtype = Q35_U8; w.shape = {ws_bytes}; w.bytes = size_t(ws_bytes);
    CUDA_OK(cudaMalloc(&w.dev, w.bytes));
    io.push_back(w);
    host_in.emplace_back();
    io.back().is_out = true;  // nothing to upload; not written to a file either (see below)
    bind();
    printf("in  %-16s %12lld bytes (scratch)\n", "workspace", (long long)ws_bytes);
  }

  // ---- first run, outputs to files
  if (upload()) return 1;
  if (q35_run(role.c_str(), call.data(), int(call.size()), nullptr)) return fail("run");
  CUDA_OK(cudaDeviceSynchronize());
  std::vector<std::vector<char>> first(io.size());
  for (size_t i = 0; i < io.size(); ++i) {
    const Entry& e = io[i];
    if (!e.is_out || e.name == "workspace") continue;
    first[i].resize(e.bytes);
    CUDA_OK(cudaMemcpy(first[i].data(), e.dev, e.bytes, cudaMemcpyDeviceToHost));
    const std::string path = dir + "/out_" + e.name + ".bin";
    std::ofstream(path, std::ios::binary).write(first[i].data(), std::streamsize(e.bytes));
    printf("out %-16s %12zu bytes -> %s\n", e.name.c_str(), e.bytes, path.c_str());
  }

  // ---- repeated runs from the same inputs must reproduce the first bit for bit
  int bad = 0;
  for (int r = 0; r < check; ++r) {
    if (upload()) return 1;
    if (q35_run(role.c_str(), call.data(), int(call.size()), nullptr)) return fail("run (check)");
    CUDA_OK(cudaDeviceSynchronize());
    for (size_t i = 0; i < io.size(); ++i) {
      if (first[i].empty()) continue;
      std::vector<char> now(io[i].bytes);
      CUDA_OK(cudaMemcpy(now.data(), io[i].dev, io[i].bytes, cudaMemcpyDeviceToHost));
      if (memcmp(now.data(), first[i].data(), io[i].bytes)) {
        ++bad;
        printf("check run %d: output %s differs from the first run\n", r, io[i].name.c_str());
      }
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
      if (q35_run(role.c_str(), call.data(), int(call.size()), nullptr)) return fail("run (timed)");
    CUDA_OK(cudaEventRecord(t1));
    CUDA_OK(cudaEventSynchronize(t1));
    float ms = 0.f;
    CUDA_OK(cudaEventElapsedTime(&ms, t0, t1));
    printf("%s: %.1f us per run over %d runs\n", role.c_str(), ms * 1e3f / float(reps), reps);
  }
  const int status = q35_device_status(nullptr);
  printf("device status %d\n", status);
  return (bad || status) ? 1 : 0;
}
