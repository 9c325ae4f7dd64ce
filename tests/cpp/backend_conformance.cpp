// The reference's matrix-product known-answer tests (Sources/HCTestUtils/BackendTests.swift:
// 684-725, 769-783) replayed through the C++ mirror of the Backend interface, followed by the
// operations either side of a Linear product on the same small exact values.  Prints
// "conformance ok" and exits 0 when every check holds.
#include <cmath>
#include <cstdio>
#include <vector>

#include "hc_cuda.hpp"

using namespace honeycrisp;

static uint16_t to_half(float f) {   // exact for the small integers used here
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if (f == 0.0f) return (uint16_t)((x >> 16) & 0x8000u);
  const uint32_t sign = (x >> 16) & 0x8000u, exp = ((x >> 23) & 0xff) - 127 + 15, man = (x >> 13) & 0x3ff;
  return (uint16_t)(sign | (exp << 10) | man);
}
static float from_half(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
  uint32_t bits;
  if (exp == 0 && man == 0) bits = sign;
  else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
  else bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

static std::shared_ptr<TensorData> upload(Backend& be, const std::vector<float>& v, DType dt) {
  if (dt == DType::float32) return be.collection(v.data(), v.size(), dt);
  std::vector<uint16_t> h(v.size());
  for (size_t i = 0; i < v.size(); i++) h[i] = to_half(v[i]);
  return be.collection(h.data(), h.size(), dt);
}
static std::vector<float> download(const std::shared_ptr<TensorData>& d, DType dt) {
  auto bytes = d->onCPU();
  std::vector<float> out(bytes.size() / byteSize(dt));
  for (size_t i = 0; i < out.size(); i++) {
    if (dt == DType::float32) std::memcpy(&out[i], &bytes[4 * i], 4);
    else { uint16_t h; std::memcpy(&h, &bytes[2 * i], 2); out[i] = from_half(h); }
  }
  return out;
}
static std::vector<float> transposed(const std::vector<float>& v, int r, int c) {
  std::vector<float> t(v.size());
  for (int i = 0; i < r; i++) for (int j = 0; j < c; j++) t[j * r + i] = v[i * c + j];
  return t;
}
#define CHECK(cond) do { if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); return 1; } } while (0)

int main() {
  CUDABackend backend(0);
  Backend& be = backend;
  const std::vector<float> x = {1, 2, 3, 4, 5, 6};                                  // [2,3]
  const std::vector<float> y43 = {-1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12};  // [4,3], used as y = y43^T [3,4]
  const std::vector<float> y = transposed(y43, 4, 3);
  const std::vector<float> expect = {-14, -32, -50, -68, -32, -77, -122, -167};
  for (int ta = 0; ta < 2; ta++) for (int tb = 0; tb < 2; tb++) for (int to = 0; to < 2; to++)
    for (DType dt : {DType::float32, DType::float16}) {
      auto a = upload(be, ta ? transposed(x, 2, 3) : x, dt);
      auto b = upload(be, tb ? transposed(y, 3, 4) : y, dt);
      auto out = be.matmul(a, ta, b, tb, to, 2, 3, 4, dt);
      out->wait();
      auto got = download(out, dt);
      if (to) got = transposed(got, 4, 2);
      CHECK(got == expect);
    }
  {  // ones[64,128] x ones[128,32] == 128; float16 finite; x1000 overflows to +inf
    std::vector<float> a(64 * 128, 1.0f), b(128 * 32, 1.0f);
    auto z = download(be.matmul(upload(be, a, DType::float32), false, upload(be, b, DType::float32), false, false, 64, 128, 32, DType::float32), DType::float32);
    for (float v : z) CHECK(v == 128.0f);
    auto s = download(be.matmul(upload(be, a, DType::float16), false, upload(be, b, DType::float16), false, false, 64, 128, 32, DType::float16), DType::float16);
    for (float v : s) CHECK(std::isfinite(v));
    std::vector<float> a1k(64 * 128, 1000.0f), b1k(128 * 32, 1000.0f);
    auto big = download(be.matmul(upload(be, a1k, DType::float16), false, upload(be, b1k, DType::float16), false, false, 64, 128, 32, DType::float16), DType::float16);
    for (float v : big) CHECK(std::isinf(v) && v > 0);
  }
  {  // matrix-vector product and its two gradients (Linalg.swift:73-80 flag algebra)
    auto xd = upload(be, x, DType::float32);
    auto yd = upload(be, {-1, -3, 2}, DType::float32);
    CHECK(download(be.matmul(xd, false, yd, false, false, 2, 3, 1, DType::float32), DType::float32) == (std::vector<float>{-1, -7}));
    auto g = upload(be, {1, 1}, DType::float32);
    CHECK(download(be.matmul(g, false, yd, true, false, 2, 1, 3, DType::float32), DType::float32) == (std::vector<float>{-1, -3, 2, -1, -3, 2}));
    CHECK(download(be.matmul(xd, true, g, false, false, 3, 2, 1, DType::float32), DType::float32) == (std::vector<float>{5, 7, 9}));
  }
  {  // batched equals per-matrix; an unimplemented dtype throws notImplemented
    std::vector<float> a(3 * 2 * 3), b(3 * 3 * 4);
    for (size_t i = 0; i < a.size(); i++) a[i] = (float)((i * 7) % 5) - 2;
    for (size_t i = 0; i < b.size(); i++) b[i] = (float)((i * 3) % 7) - 3;
    auto all = download(be.batchedMatmul(3, upload(be, a, DType::float32), false, upload(be, b, DType::float32), false, false, 2, 3, 4, DType::float32), DType::float32);
    for (int m = 0; m < 3; m++) {
      std::vector<float> am(a.begin() + m * 6, a.begin() + (m + 1) * 6), bm(b.begin() + m * 12, b.begin() + (m + 1) * 12);
      auto one = download(be.matmul(upload(be, am, DType::float32), false, upload(be, bm, DType::float32), false, false, 2, 3, 4, DType::float32), DType::float32);
      for (int i = 0; i < 8; i++) CHECK(one[i] == all[m * 8 + i]);
    }
    bool threw = false;
    try { be.matmul(upload(be, x, DType::float32), false, upload(be, y, DType::float32), false, false, 2, 3, 4, DType::int64); }
    catch (const BackendError& e) { threw = e.kind == BackendError::Kind::notImplemented; }
    CHECK(threw);
    Backend base;
    threw = false;
    try { base.matmul(nullptr, false, nullptr, false, false, 1, 1, 1, DType::float32); }
    catch (const BackendError& e) { threw = e.kind == BackendError::Kind::notImplemented; }
    CHECK(threw);
  }
  {  // asynchronous upload ordered on the device, product, asynchronous read-back
    std::vector<float> a(256 * 64), b(64 * 128), got(256 * 128, -1.0f);
    for (size_t i = 0; i < a.size(); i++) a[i] = (float)((i * 5) % 7) - 3;
    for (size_t i = 0; i < b.size(); i++) b[i] = (float)((i * 11) % 5) - 2;
    auto ad = std::make_shared<CUDAData>(backend.context(), a.size() * 4);
    auto bd = std::make_shared<CUDAData>(backend.context(), b.size() * 4);
    hc_event* ua = ad->writeFrom(a.data(), a.size() * 4);   // later work waits for the copies on the device
    hc_event* ub = bd->writeFrom(b.data(), b.size() * 4);
    auto out = std::dynamic_pointer_cast<CUDAData>(be.matmul(ad, false, bd, false, false, 256, 64, 128, DType::float32));
    CHECK(out != nullptr);
    hc_event* rd = out->readInto(got.data(), got.size() * 4);
    CHECK(hc_event_wait(rd) == HC_OK);
    CHECK(hc_event_wait(ua) == HC_OK && hc_event_wait(ub) == HC_OK);
    hc_event_destroy(rd); hc_event_destroy(ua); hc_event_destroy(ub);
    for (int i = 0; i < 256; i += 51) for (int j = 0; j < 128; j += 17) {
      float want = 0.0f;
      for (int k = 0; k < 64; k++) want += a[i * 64 + k] * b[k * 128 + j];   // small integers: exact
      CHECK(got[i * 128 + j] == want);
    }
  }
  {  // either side of a Linear product: constant, cast, linear = product + broadcast add, the bias
     // gradient (column sum), gradient accumulation (add), the materialised transpose
    for (DType dt : {DType::float32, DType::float16}) {
      auto ones = download(be.constant(1.0f, 37, dt), dt);
      CHECK(ones.size() == 37);
      for (float v : ones) CHECK(v == 1.0f);
      auto w = upload(be, y, dt);                       // [3,4]
      auto xd = upload(be, x, dt);                      // [2,3]
      auto bias = upload(be, {10, 20, 30, 40}, dt);
      auto h = download(be.linear(xd, w, bias, 2, 3, 4, dt), dt);
      for (int i = 0; i < 2; i++) for (int j = 0; j < 4; j++) CHECK(h[i * 4 + j] == expect[i * 4 + j] + 10.0f * (j + 1));
      CHECK(download(be.linear(xd, w, nullptr, 2, 3, 4, dt), dt) == expect);
      auto g = upload(be, {8, 7, 6, 5, 4, 3, 2, 1}, dt);   // upstream gradient [2,4]
      CHECK(download(be.columnSum(g, 2, 4, dt), dt) == (std::vector<float>{12, 10, 8, 6}));
      CHECK(download(be.add(g, g, 8, dt), dt) == (std::vector<float>{16, 14, 12, 10, 8, 6, 4, 2}));
      CHECK(download(be.transpose(g, 1, 2, 4, dt), dt) == transposed({8, 7, 6, 5, 4, 3, 2, 1}, 2, 4));
    }
    auto half = be.cast(upload(be, {1.5f, -2.0f, 65520.0f}, DType::float32), 3, DType::float32, DType::float16);
    auto hv = download(half, DType::float16);
    CHECK(hv[0] == 1.5f && hv[1] == -2.0f && std::isinf(hv[2]));
    CHECK(download(be.cast(half, 2, DType::float16, DType::float32), DType::float32)[0] == 1.5f);
    bool threw = false;
    try { be.constant(0.0f, 4, DType::int64); }
    catch (const BackendError& e) { threw = e.kind == BackendError::Kind::notImplemented; }
    CHECK(threw);
  }
  std::printf("conformance ok\n");
  return 0;
}
