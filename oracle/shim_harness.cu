// Test harness (checker side, not part of the product): calls the reference-named C++ launchers of
// libhelios_b200.so (include/helios_b200_shim.hpp) - the entry points the engine's layer loop would call - on
// inputs read from a directory, and writes their outputs back, so that a pytest can compare them bit for bit with
// the hk_* C ABI called through ctypes.  Usage: shim_harness <dir>; tensors are raw little-endian files <dir>/<name>.bin.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "../include/helios_b200_shim.hpp"

using namespace helios;
static std::string g_dir;

static std::vector<char> slurp(const char* name) {
  const std::string p = g_dir + "/" + name + ".bin";
  FILE* f = std::fopen(p.c_str(), "rb");
  if (!f) { std::fprintf(stderr, "missing %s\n", p.c_str()); std::exit(2); }
  std::fseek(f, 0, SEEK_END);
  const long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<char> v(n);
  if (std::fread(v.data(), 1, n, f) != (size_t)n) std::exit(2);
  std::fclose(f);
  return v;
}
static void* upload(const char* name, size_t* bytes = nullptr) {
  const std::vector<char> v = slurp(name);
  void* d = nullptr;
  if (cudaMalloc(&d, v.size() ? v.size() : 16) != cudaSuccess) std::exit(3);
  cudaMemcpy(d, v.data(), v.size(), cudaMemcpyHostToDevice);
  if (bytes) *bytes = v.size();
  return d;
}
static void* alloc(size_t bytes) {
  void* d = nullptr;
  if (cudaMalloc(&d, bytes) != cudaSuccess) std::exit(3);
  cudaMemset(d, 0, bytes);
  return d;
}
static void download(const char* name, const void* d, size_t bytes) {
  std::vector<char> v(bytes);
  if (cudaMemcpy(v.data(), d, bytes, cudaMemcpyDeviceToHost) != cudaSuccess) { std::fprintf(stderr, "copy back of %s failed\n", name); std::exit(4); }
  const std::string p = g_dir + "/out_" + name + ".bin";
  FILE* f = std::fopen(p.c_str(), "wb");
  std::fwrite(v.data(), 1, bytes, f);
  std::fclose(f);
}

int main(int argc, char** argv) {
  if (argc < 2) return 1;
  g_dir = argv[1];
  cudaSetDevice(0);
  // ---- KDA recurrence launcher: seqlen 1 (per-token kernel), 64 and 200 (chunked kernel; the launcher's scratch
  //      grows between the two), all on the same state ----
  {
    const int H = 4, D = 128, T = 265, row = 3 * H * D;
    auto* qkv = (aux::bfloat16*)upload("rec_qkv");
    auto* g = (float*)upload("rec_g");
    auto* beta = (aux::bfloat16*)upload("rec_beta");
    auto* st = (float*)upload("rec_state");
    auto* out = (aux::bfloat16*)alloc((size_t)T * H * D * 2);
    int t0 = 0;
    for (int n : {1, 64, 200}) {
      aux::cuda_recurrent_gated_delta_rule(qkv + (size_t)t0 * row, g + (size_t)t0 * H * D, beta + (size_t)t0 * H, st,
                                           out + (size_t)t0 * H * D, 1, n, H, H, D, D, 1, nullptr, true, false, nullptr);
      t0 += n;
    }
    cudaDeviceSynchronize();
    download("rec_out", out, (size_t)T * H * D * 2);
    download("rec_state", st, (size_t)H * D * D * 4);
  }
  // ---- short conv ----
  {
    const int dim = 1536, T = 37;
    auto* x = (aux::bfloat16*)upload("conv_x");
    auto* st = (aux::bfloat16*)upload("conv_state");
    auto* w = (aux::bfloat16*)upload("conv_w");
    auto* out = (aux::bfloat16*)alloc((size_t)T * dim * 2);
    aux::cuda_causal_conv1d_update(x, st, nullptr, w, nullptr, out, 1, dim, T, 4, 4, true, false, nullptr);
    cudaDeviceSynchronize();
    download("conv_out", out, (size_t)T * dim * 2);
    download("conv_state", st, (size_t)dim * 4 * 2);
  }
  // ---- top-k ----
  {
    const int R = 3, T = 1000;
    auto* sc = (half*)upload("topk_scores");
    auto* idx = (int*)alloc((size_t)R * 512 * 4);
    aux::dsa_topk(sc, T, idx, R, T, 512, 512);
    cudaDeviceSynchronize();
    download("topk_idx", idx, (size_t)R * 512 * 4);
  }
  // ---- gated RMS norm (bf16 x, bf16 weight, float gate, half out, sigmoid gate) ----
  {
    const int rows = 64, dim = 128;
    void* x = upload("norm_x");
    void* w = upload("norm_w");
    void* g = upload("norm_g");
    void* y = alloc((size_t)rows * dim * 2);
    aux::gated_rms_norm(x, w, aux::kBFloat16, y, aux::kHalf, g, aux::kFloat, rows, dim, 1e-6f, 0.0f, 1, false, 1);
    cudaDeviceSynchronize();
    download("norm_y", y, (size_t)rows * dim * 2);
  }
  // ---- KDA producers ----
  {
    const int S = 33, H = 4, Dk = 128, F = 3 * H * Dk;
    auto* qkv = (float*)upload("prep_qkv");
    auto* b = (float*)upload("prep_b");
    auto* f = (float*)upload("prep_f");
    auto* dtb = (float*)upload("prep_dt_bias");
    auto* alog = (float*)upload("prep_a_log");
    void* mixed = alloc((size_t)F * S * 2);
    void* beta = alloc((size_t)S * H * 2);
    auto* g = (float*)alloc((size_t)S * H * Dk * 4);
    glue::kda_transpose_cast(mixed, qkv, S, F);
    glue::kda_gate(b, f, dtb, alog, -5.0f, beta, g, S, H, Dk);
    cudaDeviceSynchronize();
    download("prep_mixed", mixed, (size_t)F * S * 2);
    download("prep_beta", beta, (size_t)S * H * 2);
    download("prep_g", g, (size_t)S * H * Dk * 4);
    void* mixed2 = alloc((size_t)F * S * 2);
    void* beta2 = alloc((size_t)S * H * 2);
    auto* g2 = (float*)alloc((size_t)S * H * Dk * 4);
    glue::kda_prepare(qkv, b, f, dtb, alog, -5.0f, mixed2, beta2, g2, S, F, H, Dk);
    cudaDeviceSynchronize();
    download("prep2_mixed", mixed2, (size_t)F * S * 2);
    download("prep2_beta", beta2, (size_t)S * H * 2);
    download("prep2_g", g2, (size_t)S * H * Dk * 4);
  }
  b200::release_scratch();
  if (cudaDeviceSynchronize() != cudaSuccess) return 5;
  std::puts("SHIM HARNESS DONE");
  return 0;
}
