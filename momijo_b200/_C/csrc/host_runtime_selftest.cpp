// Self-test driver for the host runtime (host_runtime.cpp), meant to be built together with it under
// AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer (see build.build_sanitized):
// it drives every exported entry point, the multi-threaded blob reader with 1..8 threads and several
// concurrent callers included, checks the results, and exits non-zero on a mismatch. The sanitizers
// turn out-of-bounds accesses, leaks, integer overflow and data races into a non-zero exit as well.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
long long mmj_blob_write(const char* path, const void* src, long long nbytes, long long offset, int truncate);
long long mmj_blob_read(const char* path, void* dst, long long nbytes, long long offset, int threads);
long long mmj_file_size(const char* path);
long long mmj_pack_csv_f32(const float* x, long long n, char* out, long long cap);
long long mmj_unpack_csv_f32(const char* s, long long len, float* out, long long cap);
void mmj_lcg_shuffle(long long* idx, long long n, unsigned int seed);
unsigned long long mmj_fnv1a64(const unsigned char* data, long long n);
void mmj_cpu_resize_nearest_u8(const unsigned char* src, int H, int W, int C, unsigned char* dst, int OH, int OW);
void mmj_cpu_rgb_to_gray_u8(const unsigned char* src, long long npix, unsigned char* dst);
void mmj_cpu_resize_bilinear_u8(const unsigned char* src, int H, int W, int C, unsigned char* dst, int OH, int OW);
}

static int failures = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::fprintf(stderr, "selftest: %s failed (line %d)\n", #cond, __LINE__); \
      ++failures;                                                          \
    }                                                                      \
  } while (0)

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : "/tmp";
  const std::string path = dir + "/mmj_selftest.bin";

  // blob write / read: 20 MiB written in two pieces, read back with 1..8 threads at odd offsets
  const long long n = (20ll << 20) + 12345;
  std::vector<unsigned char> src((size_t)n);
  for (long long i = 0; i < n; ++i) src[(size_t)i] = (unsigned char)((i * 131 + (i >> 9)) & 255);
  CHECK(mmj_blob_write(path.c_str(), src.data(), n / 2, 0, 1) == 0);
  CHECK(mmj_blob_write(path.c_str(), src.data() + n / 2, n - n / 2, n / 2, 0) == 0);
  CHECK(mmj_file_size(path.c_str()) == n);
  for (int threads = 1; threads <= 8; ++threads) {
    const long long off = 1000 + 7 * threads, len = n - off - 3;
    std::vector<unsigned char> dst((size_t)len);
    CHECK(mmj_blob_read(path.c_str(), dst.data(), len, off, threads) == len);
    CHECK(std::memcmp(dst.data(), src.data() + off, (size_t)len) == 0);
  }
  // several callers at once (each call spawns its own readers)
  {
    std::atomic<int> bad{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < 4; ++t)
      ts.emplace_back([&, t] {
        const long long off = 4096ll * t, len = (9ll << 20);
        std::vector<unsigned char> dst((size_t)len);
        if (mmj_blob_read(path.c_str(), dst.data(), len, off, 3) != len) ++bad;
        if (std::memcmp(dst.data(), src.data() + off, (size_t)len) != 0) ++bad;
      });
    for (auto& t : ts) t.join();
    CHECK(bad.load() == 0);
  }
  CHECK(mmj_blob_read((path + ".missing").c_str(), src.data(), 16, 0, 2) < 0);
  CHECK(mmj_file_size((path + ".missing").c_str()) == -1);
  std::remove(path.c_str());

  // CSV packing: round trip, and the "capacity too small" answer
  {
    std::vector<float> x = {0.f, -1.5f, 3.14159274f, 1e-20f, -2.5e30f, 123456.789f};
    char small[4];
    const long long need = mmj_pack_csv_f32(x.data(), (long long)x.size(), small, sizeof(small));
    CHECK(need < 0);
    std::vector<char> buf((size_t)(-need) + 8);
    const long long len = mmj_pack_csv_f32(x.data(), (long long)x.size(), buf.data(), (long long)buf.size());
    CHECK(len > 0);
    std::vector<float> y(x.size() + 2, 0.f);
    CHECK(mmj_unpack_csv_f32(buf.data(), len, y.data(), (long long)y.size()) == (long long)x.size());
    for (size_t i = 0; i < x.size(); ++i) CHECK(x[i] == y[i]);
    CHECK(mmj_unpack_csv_f32(buf.data(), len, y.data(), 2) >= 2);   // a short output buffer is never overrun
  }

  // shuffle: a permutation, reproducible per seed
  {
    const long long m = 1000;
    std::vector<long long> a((size_t)m), b((size_t)m), c((size_t)m);
    mmj_lcg_shuffle(a.data(), m, 7u);
    mmj_lcg_shuffle(b.data(), m, 7u);
    mmj_lcg_shuffle(c.data(), m, 8u);
    CHECK(a == b);
    CHECK(a != c);
    std::vector<int> seen((size_t)m, 0);
    for (long long v : a) {
      CHECK(v >= 0 && v < m);
      if (v >= 0 && v < m) ++seen[(size_t)v];
    }
    for (int s : seen) CHECK(s == 1);
    mmj_lcg_shuffle(a.data(), 0, 1u);
    mmj_lcg_shuffle(a.data(), 1, 1u);
  }

  // hash and the image loops (odd sizes, up- and down-scaling)
  {
    const unsigned char t[] = "momijo";
    CHECK(mmj_fnv1a64(t, 6) != mmj_fnv1a64(t, 5));
    CHECK(mmj_fnv1a64(t, 0) == 1469598103934665603ull);
    const int H = 37, W = 53, C = 3;
    std::vector<unsigned char> img((size_t)H * W * C);
    for (size_t i = 0; i < img.size(); ++i) img[i] = (unsigned char)(i * 7);
    std::vector<unsigned char> gray((size_t)H * W);
    mmj_cpu_rgb_to_gray_u8(img.data(), (long long)H * W, gray.data());
    CHECK(gray[0] == (unsigned char)((299 * img[0] + 587 * img[1] + 114 * img[2]) / 1000));
    for (int oh : {1, 19, 37, 80})
      for (int ow : {1, 31, 53, 97}) {
        std::vector<unsigned char> a((size_t)oh * ow * C), b((size_t)oh * ow * C);
        mmj_cpu_resize_nearest_u8(img.data(), H, W, C, a.data(), oh, ow);
        mmj_cpu_resize_bilinear_u8(img.data(), H, W, C, b.data(), oh, ow);
        CHECK(a[0] == img[0]);
      }
  }

  if (failures) {
    std::fprintf(stderr, "selftest: %d check(s) failed\n", failures);
    return 1;
  }
  std::puts("host runtime selftest ok");
  return 0;
}
