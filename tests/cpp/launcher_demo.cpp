// A few of the reference engine's launch sites written with the reference's own launcher
// names (include/gptoss_launchers.hpp), driven from files so that a test can compare the
// outcome with direct calls through the C ABI.
//   launcher_demo <in.bin> <out.bin>
// in.bin : int32 B, H, E, k, slots, slot | x[B,H] f32 | y[B,H] f32 | w[H] f32 | qkv[B,5120] f32 |
//          cos[32] f32 | sin[32] f32 | logits[B,E] f32 | Z[B*k,H] f32
// out.bin: x_after_add[B,H] f32 | t16[B,H] u16 | qkv_after[B,5120] f32 | kc | vq | vs |
//          topk_w[B,k] f32 | topk_e[B,k] i32 | x_after_combine[B,H] f32 | t16_after_combine[B,H] u16
#include <stdio.h>

#include <vector>

#include "gptoss_engine.h"
#include "gptoss_launchers.hpp"

using namespace gptoss_ref_names;

template <typename T> static T *to_device(const std::vector<T> &h) {
  void *p = nullptr;
  GPTOSS_CHECK(gptoss_device_alloc(&p, h.size() * sizeof(T)));
  GPTOSS_CHECK(gptoss_upload(p, h.data(), h.size() * sizeof(T), nullptr));
  return static_cast<T *>(p);
}
template <typename T> static T *device_fill(size_t n, int byte) {
  void *p = nullptr;
  GPTOSS_CHECK(gptoss_device_alloc(&p, n * sizeof(T)));
  GPTOSS_CHECK(gptoss_device_memset(p, byte, n * sizeof(T), nullptr));
  return static_cast<T *>(p);
}
template <typename T> static void dump(FILE *f, const T *dev, size_t n) {
  std::vector<T> h(n);
  GPTOSS_CHECK(gptoss_device_synchronize());
  GPTOSS_CHECK(gptoss_download(h.data(), dev, n * sizeof(T), nullptr));
  GPTOSS_CHECK(gptoss_device_synchronize());
  fwrite(h.data(), sizeof(T), n, f);
}
template <typename T> static std::vector<T> slurp(FILE *f, size_t n) {
  std::vector<T> v(n);
  if (fread(v.data(), sizeof(T), n, f) != n) {
    fprintf(stderr, "short read\n");
    exit(2);
  }
  return v;
}

int main(int argc, char **argv) {
  if (argc != 3)
    return 2;
  FILE *in = fopen(argv[1], "rb"), *out = fopen(argv[2], "wb");
  if (!in || !out)
    return 2;
  const std::vector<int> dims = slurp<int>(in, 6);
  const int B = dims[0], H = dims[1], E = dims[2], k = dims[3], slots = dims[4], slot = dims[5];
  const int NQ = 64, NKV = 8, QKV = (NQ + 2 * NKV) * 64;
  GPTOSS_CHECK(gptoss_device_set(0));
  float *x = to_device(slurp<float>(in, (size_t)B * H));
  float *y = to_device(slurp<float>(in, (size_t)B * H));
  float *w = to_device(slurp<float>(in, H));
  float *qkv = to_device(slurp<float>(in, (size_t)B * QKV));
  float *cosv = to_device(slurp<float>(in, 32)), *sinv = to_device(slurp<float>(in, 32));
  float *logits = to_device(slurp<float>(in, (size_t)B * E));
  float *Z = to_device(slurp<float>(in, (size_t)B * k * H));
  bf16_t *t16 = device_fill<bf16_t>((size_t)B * H, 0);
  const size_t kv = (size_t)B * slots * NKV * 64;
  bf16_t *kc = device_fill<bf16_t>(kv, 0x55);
  int8_t *vq = device_fill<int8_t>(kv, 0x55);
  float *vs = device_fill<float>(kv / 64, 0x55);
  float *topk_w = device_fill<float>((size_t)B * k, 0);
  int *topk_e = device_fill<int>((size_t)B * k, 0);
  gptoss_stream_t s = nullptr;

  add_rmsnorm_bf16(s, B, x, y, w, t16, H);                                        // gpu_engine.hpp:503
  dump(out, x, (size_t)B * H);
  dump(out, t16, (size_t)B * H);
  rope_kv_bf16(s, B, qkv, QKV, cosv, sinv, NQ, NKV, kc, vq, vs, slots, slot, false); // :495
  dump(out, qkv, (size_t)B * QKV);
  dump(out, kc, kv);
  dump(out, vq, kv);
  dump(out, vs, kv / 64);
  router_topk_wave(s, logits, E, k, topk_w, topk_e, B, nullptr, nullptr);           // :525
  dump(out, topk_w, (size_t)B * k);
  dump(out, topk_e, (size_t)B * k);
  moe_combine_rmsnorm(s, B, x, Z, nullptr, topk_w, topk_e, k, H, w, t16);           // :602
  dump(out, x, (size_t)B * H);
  dump(out, t16, (size_t)B * H);
  fclose(in);
  fclose(out);
  return 0;
}
