// Standalone check of the narrow-float decodes every weight-streaming kernel relies on
// (common.cuh): all 256 byte values of packed e2m1 pairs through cvt.rn.f16x2.e2m1x2 and all
// 256 e4m3 bytes through cvt.rn.f16x2.e4m3x2, against tables computed on the host from the
// format definitions.  Exit code 0 and "ok" when every value matches exactly.
// Counterpart of the reference's scripts/_test_prmt_standalone.cu (its prmt-based nibble decode).
//   nvcc -gencode arch=compute_100a,code=sm_100a -o narrow_decode csrc/tests/narrow_decode.cu
#include <cmath>
#include <cstdio>

#include "../common.cuh"

__global__ void decode_kernel(float* e2m1_out /*[256][2]*/, float* e4m3_out /*[256]*/) {
  const int b = threadIdx.x;   // 256 threads, one byte value each
  uint32_t h[4];
  cvt_e2m1x8_to_h2x4((uint32_t)b | ((uint32_t)b << 8) | ((uint32_t)b << 16) | ((uint32_t)b << 24), h);
  const float2 v0 = h2_to_f2(h[0]), v3 = h2_to_f2(h[3]);
  // the four byte lanes carry the same byte: lanes 0 and 3 must agree
  e2m1_out[2 * b] = (v0.x == v3.x) ? v0.x : NAN;
  e2m1_out[2 * b + 1] = (v0.y == v3.y) ? v0.y : NAN;
  const float2 s = h2_to_f2(cvt_e4m3x2_to_h2((uint16_t)(b | (((b + 1) & 0xFF) << 8))));
  e4m3_out[b] = s.x;   // low byte -> low half
  // the high half is the decode of byte b + 1: checked through the next thread's low half
  (void)s.y;
}

static float host_e2m1(int nib) {
  static const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = lut[nib & 7];
  return (nib & 8) ? -v : v;
}

static float host_e4m3(int b) {
  const int sign = b >> 7, e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7) return NAN;                       // the one NaN pattern of e4m3fn
  if (e == 0) v = std::ldexp((float)m / 8.f, -6);          // subnormal
  else v = std::ldexp(1.f + (float)m / 8.f, e - 7);
  return sign ? -v : v;
}

int main() {
  float *d2, *d4, h2[512], h4[256];
  if (cudaMalloc(&d2, sizeof(h2)) != cudaSuccess || cudaMalloc(&d4, sizeof(h4)) != cudaSuccess) {
    std::printf("no device memory\n");
    return 2;
  }
  decode_kernel<<<1, 256>>>(d2, d4);
  if (cudaMemcpy(h2, d2, sizeof(h2), cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(h4, d4, sizeof(h4), cudaMemcpyDeviceToHost) != cudaSuccess) {
    std::printf("kernel failed: %s\n", cudaGetErrorString(cudaGetLastError()));
    return 2;
  }
  int bad = 0;
  for (int b = 0; b < 256; ++b) {
    const float lo = host_e2m1(b & 15), hi = host_e2m1(b >> 4);   // low nibble = even element
    if (!(h2[2 * b] == lo) || !(h2[2 * b + 1] == hi)) {
      if (bad++ < 8) std::printf("e2m1 byte %02x: got (%g, %g) want (%g, %g)\n", b, h2[2 * b], h2[2 * b + 1], lo, hi);
    }
    const float w = host_e4m3(b);
    const bool same = std::isnan(w) ? std::isnan(h4[b]) : (h4[b] == w);
    if (!same) {
      if (bad++ < 8) std::printf("e4m3 byte %02x: got %g want %g\n", b, h4[b], w);
    }
  }
  cudaFree(d2);
  cudaFree(d4);
  std::printf(bad ? "FAILED: %d mismatches\n" : "ok\n", bad);
  return bad ? 1 : 0;
}
