// Reader and writer of the EXL3 expert tensors of a compiled-model artifact, and the binder that turns them into the
// descriptor table the kernels index as (layer*64+expert)*3+part.
//
// Format (the reference's, src/model/compiled.cpp:91-216): a directory with `manifest.json` and `weights.bin`.  The
// manifest names every tensor with its shape [rows = outputs, cols = inputs], its format ("EXL3_K3" | "EXL3_K4" |
// "EXL3_K6"), `"codebook": "mul1"`, `"hadamard_block": 128` and three byte regions of the payload: `packed`
// (rows*cols*rate/8 bytes of trellis tiles), `suh` (2*cols bytes of FP16) and `svh` (2*rows bytes).  Regions start on
// 256-byte boundaries, lie back to back in offset order (each at the previous end rounded up to 256) and account for
// every payload byte; sidecar values are finite and non-zero; the payload's SHA-256 is recorded.  Expert tensors are
// named model.layers.<L>.mlp.experts.<E>.{gate,up,down}_proj.weight (src/cuda/inference.cu:1599-1602).
//
// Scope: the expert tensors only.  The reference's manifest also carries attention, embedding and head tensors,
// tokenizer and model-revision identities; a reader of whole checkpoints passes `experts_only = true` to skip tensors
// that are not expert tensors instead of rejecting them.
#pragma once
#include <cstdint>
#include <filesystem>
#include <map>
#include <string>
#include <vector>

#include "../../include/padra_b200.h"

namespace padra_b200::artifact {

struct Region {
  std::uint64_t offset = 0, bytes = 0;
};
struct Tensor {
  std::string name;
  int rows = 0, cols = 0, rate = 0;
  Region packed, suh, svh;
};
struct Artifact {
  std::filesystem::path directory;
  std::string profile; // mellum16-exl3-k{3,4,6}-fp8-bf16-v1 (src/model/compiled.h:11-14)
  int rate = 0;
  std::uint64_t weights_bytes = 0;
  std::string weights_sha256;
  std::map<std::string, Tensor> tensors;
  int layers = 0; // 1 + the largest layer index among the expert tensors
};

int FormatOfRate(int rate);               // 3 -> 6, 4 -> 3, 6 -> 5 (src/cuda/device_matrix.cuh:30-44)
std::string ProfileOfRate(int rate);      // src/model/compiled.h:11-14
std::string ExpertTensorName(int layer, int expert, int part);
std::string Sha256Hex(const void *data, std::size_t bytes);

// Parses and validates <directory>/manifest.json against <directory>/weights.bin; throws std::runtime_error with the
// reference loader's wording where it has one.  verify_payload also reads the payload: its hash and its sidecar values.
Artifact Load(const std::filesystem::path &directory, bool verify_payload = true, bool experts_only = false);

// One tensor's bytes for Write.
struct TensorBytes {
  std::string name;
  int rows = 0, cols = 0;
  const unsigned char *packed = nullptr;
  const std::uint16_t *suh = nullptr, *svh = nullptr;
};
// Writes weights.bin (regions in the given order, canonical 256-byte layout) and manifest.json.
void Write(const std::filesystem::path &directory, int rate, const std::vector<TensorBytes> &tensors);

// The descriptor table for `layers` layers of 64 experts x {gate, up, down}: table[(layer*64+expert)*3+part], with
// pointers into `arena`, the address at which the payload's byte 0 lives (device memory for the kernels).  Throws if a
// tensor is missing or its region lies outside `arena_bytes` (src/cuda/device_matrix.cuh:14-66).
std::vector<padra_matrix> Bind(const Artifact &artifact, const unsigned char *arena, std::uint64_t arena_bytes);

} // namespace padra_b200::artifact
