// Seeded synthetic data: a counter-based generator that gives bit-identical values on the host (numpy twin in
// seq2seqsharp_b200/synthetic.py) and on the device, so any shard of any tensor can be produced where it is used.
//   base      = splitmix64(seed ^ name_hash)
//   a, b      = splitmix64(base + 2i), splitmix64(base + 2i + 1)
//   S         = sum of the eight 16-bit fields of a and b          (Irwin-Hall, mean 262140, sigma 53509.9199...)
//   value(i)  = float( (S - 262140) * ((double)std / 53509.91992145008) )      then rounded to half for F16
#include "kernels.cuh"

namespace tsb {

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  uint64_t z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__host__ __device__ __forceinline__ float synth_value(uint64_t base, uint64_t i, double scale) {
  const uint64_t a = splitmix64(base + 2 * i), b = splitmix64(base + 2 * i + 1);
  int s = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) s += (int)((a >> (16 * k)) & 0xFFFF) + (int)((b >> (16 * k)) & 0xFFFF);
  return (float)((double)(s - 262140) * scale);
}

template <typename T>
__global__ void synth_kernel(T* __restrict__ out, int64_t n, uint64_t base, double scale) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = from_f<T>(synth_value(base, (uint64_t)i, scale));
}

int launch_synthetic(int device, DeviceState* st, void* data, int dtype, int64_t n, uint64_t seed, uint64_t name_hash,
                     float std, cudaStream_t s) {
  if (n == 0) return 1;
  const uint64_t base = splitmix64(seed ^ name_hash);
  const double scale = (double)std / 53509.91992145008;
  int64_t g = (n + 255) / 256;
  if (g > (int64_t)st->sm_count * 16) g = (int64_t)st->sm_count * 16;
  if (dtype == TSB200_F32) synth_kernel<float><<<(int)g, 256, 0, s>>>((float*)data, n, base, scale);
  else if (dtype == TSB200_F16) synth_kernel<__half><<<(int)g, 256, 0, s>>>((__half*)data, n, base, scale);
  else TSB_FAIL("fill_synthetic: unsupported dtype %d", dtype);
  count_launch(device);
  return check_launch("fill_synthetic");
}

uint64_t fnv1a64(const char* s) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (; *s; ++s) {
    h ^= (unsigned char)*s;
    h *= 0x100000001b3ull;
  }
  return h;
}

}  // namespace tsb

using namespace tsb;

extern "C" int TSB200_FillSynthetic(int device, void* data, int dtype, int64_t n, uint64_t seed, uint64_t name_hash,
                                    float std, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(data && n >= 0, "fill_synthetic: bad arguments");
  return launch_synthetic(device, st, data, dtype, n, seed, name_hash, std, pick_stream(st, stream));
}
