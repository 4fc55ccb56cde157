// Test infrastructure: converts float32 values with NVIDIA's host-side
// conversion routines (cuda_fp8.h / cuda_fp4.h) so that the numpy converters in
// nvfp4_oracle.py can be pinned against them on a machine without a GPU.
//
//   cvt_check <in.f32> <out.u8>
// writes, for every input float, two bytes: E4M3 (satfinite, RN-even) and the
// E2M1 nibble (RN-even, saturating).
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_fp8.h>
#include <cuda_fp4.h>

int main(int argc, char** argv) {
  if (argc != 3) { std::fprintf(stderr, "usage: cvt_check in.f32 out.u8\n"); return 2; }
  FILE* fi = std::fopen(argv[1], "rb");
  if (!fi) { std::perror("open input"); return 1; }
  std::fseek(fi, 0, SEEK_END);
  long bytes = std::ftell(fi);
  std::fseek(fi, 0, SEEK_SET);
  std::vector<float> x(bytes / sizeof(float));
  if (std::fread(x.data(), sizeof(float), x.size(), fi) != x.size()) return 1;
  std::fclose(fi);
  std::vector<unsigned char> out(2 * x.size());
  for (size_t i = 0; i < x.size(); ++i) {
    out[2 * i] = (unsigned char)__nv_cvt_float_to_fp8(x[i], __NV_SATFINITE, __NV_E4M3);
    out[2 * i + 1] = (unsigned char)__nv_cvt_float_to_fp4(x[i], __NV_E2M1, cudaRoundNearest);
  }
  FILE* fo = std::fopen(argv[2], "wb");
  if (!fo) { std::perror("open output"); return 1; }
  std::fwrite(out.data(), 1, out.size(), fo);
  std::fclose(fo);
  return 0;
}
