// A C++ host of the library, above its C ABI: what a maintainer of the reference's C++ runtime would write.
//
//   padra_host_tool check  <artifact dir>
//       loads and validates the artifact's expert tensors (manifest.json + weights.bin) and prints a one-line summary
//   padra_host_tool decode <artifact dir> <inputs.bin> <output.bin>
//       uploads the payload, binds the descriptor table, and runs one whole decode layer (padra_exl3_moe_decode_layer
//       through the forwarder of bind.hpp's shape, but with the artifact's own dimensions) on the current device
//
// inputs.bin: int32 layer, tokens, hidden, inter; int32 ids[tokens*8]; float routing[tokens*8];
//             float normalized[tokens*hidden]; float x[tokens*hidden]      (little endian, no padding)
// output.bin: float x[tokens*hidden] after the layer; int32 bad
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "artifact.hpp"

namespace {

namespace art = padra_b200::artifact;

void Cuda(cudaError_t e, const char *what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void Check(int status, const char *what) {
  if (status != PADRA_OK)
    throw std::runtime_error(std::string(what) + ": " + padra_status_string(status));
}
template <typename T> struct DeviceBuffer {
  T *p = nullptr;
  std::size_t n = 0;
  explicit DeviceBuffer(std::size_t count) : n(count) { Cuda(cudaMalloc(reinterpret_cast<void **>(&p), count * sizeof(T)), "cudaMalloc"); }
  ~DeviceBuffer() { cudaFree(p); }
  DeviceBuffer(const DeviceBuffer &) = delete;
  DeviceBuffer &operator=(const DeviceBuffer &) = delete;
  void Upload(const T *host, cudaStream_t s) { Cuda(cudaMemcpyAsync(p, host, n * sizeof(T), cudaMemcpyHostToDevice, s), "upload"); }
  void Download(T *host, cudaStream_t s) { Cuda(cudaMemcpyAsync(host, p, n * sizeof(T), cudaMemcpyDeviceToHost, s), "download"); }
};

std::vector<char> ReadAll(const std::string &path) {
  std::ifstream in(path, std::ios::binary | std::ios::ate);
  if (!in)
    throw std::runtime_error("cannot open " + path);
  std::vector<char> bytes(static_cast<std::size_t>(in.tellg()));
  in.seekg(0);
  in.read(bytes.data(), static_cast<std::streamsize>(bytes.size()));
  return bytes;
}

int RunCheck(const std::string &dir) {
  const art::Artifact a = art::Load(dir);
  std::cout << "{\"profile\": \"" << a.profile << "\", \"rate\": " << a.rate << ", \"layers\": " << a.layers
            << ", \"tensors\": " << a.tensors.size() << ", \"weights_bytes\": " << a.weights_bytes << ", \"weights_sha256\": \""
            << a.weights_sha256 << "\"}" << std::endl;
  return 0;
}

int RunDecode(const std::string &dir, const std::string &inputs_path, const std::string &output_path) {
  const art::Artifact a = art::Load(dir);
  const std::vector<char> in = ReadAll(inputs_path);
  if (in.size() < 16)
    throw std::runtime_error("inputs.bin too short");
  int header[4];
  std::memcpy(header, in.data(), 16);
  const int layer = header[0], tokens = header[1], hidden = header[2], inter = header[3];
  if (tokens < 1 || tokens > 16 || layer < 0 || layer >= a.layers)
    throw std::runtime_error("inputs.bin: layer or token count out of range");
  const std::size_t pairs = static_cast<std::size_t>(tokens) * 8, row = static_cast<std::size_t>(tokens) * hidden;
  if (in.size() != 16 + pairs * 4 + pairs * 4 + row * 4 * 2)
    throw std::runtime_error("inputs.bin has the wrong size for its header");
  const auto *ids = reinterpret_cast<const int *>(in.data() + 16);
  const auto *routing = reinterpret_cast<const float *>(in.data() + 16 + pairs * 4);
  const auto *normalized = routing + pairs;
  const auto *x = normalized + row;
  const art::Tensor &gate = a.tensors.at(art::ExpertTensorName(layer, 0, 0));
  if (gate.rows != inter || gate.cols != hidden)
    throw std::runtime_error("inputs.bin dimensions do not match the artifact");

  Check(padra_device_supported(), "padra_device_supported");
  cudaStream_t stream;
  Cuda(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
  const std::vector<char> payload = ReadAll((a.directory / "weights.bin").string());
  DeviceBuffer<unsigned char> arena(payload.size());
  arena.Upload(reinterpret_cast<const unsigned char *>(payload.data()), stream);
  const std::vector<padra_matrix> table = art::Bind(a, arena.p, payload.size());
  DeviceBuffer<padra_matrix> descriptors(table.size());
  descriptors.Upload(table.data(), stream);

  DeviceBuffer<int> d_ids(pairs), d_bad(1);
  DeviceBuffer<float> d_routing(pairs), d_normalized(row), d_x(row);
  DeviceBuffer<unsigned short> d_table(65536);
  d_ids.Upload(ids, stream), d_routing.Upload(routing, stream), d_normalized.Upload(normalized, stream), d_x.Upload(x, stream);
  Cuda(cudaMemsetAsync(d_bad.p, 0, sizeof(int), stream), "memset");
  Check(padra_exl3_silu_build(d_table.p, stream), "padra_exl3_silu_build");
  const std::size_t workspace_bytes = padra_exl3_moe_decode_workspace_bytes(tokens, hidden, inter);
  if (!workspace_bytes)
    throw std::runtime_error("unsupported shape");
  DeviceBuffer<unsigned char> workspace(workspace_bytes);
  Check(padra_exl3_moe_decode_workspace_init(workspace.p, workspace_bytes, stream), "padra_exl3_moe_decode_workspace_init");
  Check(padra_exl3_moe_decode_layer(descriptors.p, layer, d_ids.p, d_routing.p, d_normalized.p, d_x.p, tokens, a.rate, hidden, inter,
                                    d_table.p, workspace.p, workspace_bytes, d_bad.p, stream),
        "padra_exl3_moe_decode_layer");
  std::vector<float> out(row);
  int bad = 0;
  d_x.Download(out.data(), stream);
  d_bad.Download(&bad, stream);
  Cuda(cudaStreamSynchronize(stream), "synchronize");
  Cuda(cudaStreamDestroy(stream), "cudaStreamDestroy");
  std::ofstream result(output_path, std::ios::binary | std::ios::trunc);
  result.write(reinterpret_cast<const char *>(out.data()), static_cast<std::streamsize>(row * 4));
  result.write(reinterpret_cast<const char *>(&bad), 4);
  if (!result.good())
    throw std::runtime_error("cannot write " + output_path);
  std::cout << "{\"tokens\": " << tokens << ", \"layer\": " << layer << ", \"bad\": " << bad << "}" << std::endl;
  return bad ? 3 : 0;
}

} // namespace

int main(int argc, char **argv) {
  try {
    const std::string command = argc > 1 ? argv[1] : "";
    if (command == "check" && argc == 3)
      return RunCheck(argv[2]);
    if (command == "decode" && argc == 5)
      return RunDecode(argv[2], argv[3], argv[4]);
    std::cerr << "usage: padra_host_tool check <artifact dir> | decode <artifact dir> <inputs.bin> <output.bin>" << std::endl;
    return 2;
  } catch (const std::exception &e) {
    std::cerr << "error: " << e.what() << std::endl;
    return 1;
  }
}
