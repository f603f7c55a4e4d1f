// Host-only driver around two UNMODIFIED pieces of the reference (anvai-labs/inferflux):
//   parse FILE      SafetensorsParser (runtime/backends/cuda/native/safetensors_parser.cpp:144-303) on a
//                   safetensors file; prints one JSON object with every tensor it found (dtype, shape,
//                   offset in the data section, byte size, an FNV-1a hash of the bytes its data_ptr maps)
//   kvplan L KV D E EstimateKvBytesPerTokenPerSequence (kv_cache_planner.h:22-37)
// This file is not reference code; it owns no parsing and no arithmetic.
#include "runtime/backends/cuda/native/kv_cache_planner.h"
#include "runtime/backends/cuda/native/safetensors_parser.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

static unsigned long long fnv1a(const unsigned char *p, size_t n) {
  unsigned long long h = 1469598103934665603ULL;
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= 1099511628211ULL;
  }
  return h;
}

int main(int argc, char **argv) {
  if (argc >= 3 && std::strcmp(argv[1], "parse") == 0) {
    inferflux::SafetensorsParser parser(argv[2]);
    if (!parser.Parse()) {
      std::printf("{\"ok\": false}\n");
      return 1;
    }
    auto names = parser.GetTensorNames();
    std::sort(names.begin(), names.end());
    std::printf("{\"ok\": true, \"file_size\": %zu, \"tensors\": {", parser.GetFileSize());
    bool first = true;
    for (const auto &n : names) {
      const auto *t = parser.GetTensor(n);
      std::printf("%s\"%s\": {\"dtype\": \"%s\", \"shape\": [", first ? "" : ", ", n.c_str(), t->dtype.c_str());
      for (size_t i = 0; i < t->shape.size(); ++i) std::printf("%s%zu", i ? ", " : "", t->shape[i]);
      std::printf("], \"offset\": %zu, \"byte_size\": %zu, \"fnv1a\": \"%llx\"}", t->offset, t->byte_size,
                  t->data_ptr ? fnv1a(static_cast<const unsigned char *>(t->data_ptr), t->byte_size) : 0ULL);
      first = false;
    }
    std::printf("}}\n");
    return 0;
  }
  if (argc >= 6 && std::strcmp(argv[1], "kvplan") == 0) {
    const size_t per = inferflux::runtime::cuda::native::EstimateKvBytesPerTokenPerSequence(
        std::atoi(argv[2]), std::atoi(argv[3]), std::atoi(argv[4]), static_cast<size_t>(std::atoi(argv[5])));
    std::printf("{\"bytes_per_token\": %zu}\n", per);
    return 0;
  }
  std::fprintf(stderr, "usage: ref_host_probe parse FILE | kvplan LAYERS KV_HEADS HEAD_DIM ELEMENT_BYTES\n");
  return 2;
}
