// Host-side runtime (no CUDA): checkpoint blob I/O with large aligned chunks, ASCII CSV
// pack/unpack of float vectors (the text "blob" of the reference's layout B,
// legacy/src/momijo/learn/utils/tensor_bytes.mojo:40-85), the LCG Fisher-Yates shuffle shared by
// the data loaders (legacy/src/momijo/learn/data/dataset.mojo:570-597), FNV-1a hashing for the
// hub download cache (legacy/src/momijo/learn/hub/download.mojo:311), and the CPU restatements
// of the vision kernels used as oracles and timed baselines
// (legacy/src/momijo/vision/backend/cpu/resize_cpu.mojo:22-55, convert_color_cpu.mojo:45).
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>
#include <fcntl.h>
#include <unistd.h>

#define HAPI extern "C" __attribute__((visibility("default")))

// ---- blob I/O --------------------------------------------------------------------------------
// Writes `nbytes` from `src` at `offset` of `path` (created if needed). Returns 0 or -errno.
HAPI long long mmj_blob_write(const char* path, const void* src, long long nbytes, long long offset,
                              int truncate) {
  int flags = O_WRONLY | O_CREAT | (truncate ? O_TRUNC : 0);
  int fd = ::open(path, flags, 0644);
  if (fd < 0) return -errno;
  const char* p = static_cast<const char*>(src);
  long long done = 0;
  const long long chunk = 64ll << 20;
  while (done < nbytes) {
    long long n = nbytes - done < chunk ? nbytes - done : chunk;
    ssize_t w = ::pwrite(fd, p + done, (size_t)n, (off_t)(offset + done));
    if (w < 0) {
      if (errno == EINTR) continue;
      int e = errno;
      ::close(fd);
      return -e;
    }
    done += w;
  }
  ::close(fd);
  return 0;
}

// Reads `nbytes` at `offset` into `dst` with `threads` parallel preads. Returns bytes read or -errno.
HAPI long long mmj_blob_read(const char* path, void* dst, long long nbytes, long long offset,
                             int threads) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -errno;
  if (threads < 1) threads = 1;
  if (nbytes < (8ll << 20)) threads = 1;
  std::vector<long long> got(threads, 0);
  std::vector<int> err(threads, 0);
  auto work = [&](int t) {
    long long per = (nbytes + threads - 1) / threads;
    long long lo = per * t, hi = lo + per > nbytes ? nbytes : lo + per;
    char* p = static_cast<char*>(dst);
    while (lo < hi) {
      ssize_t r = ::pread(fd, p + lo, (size_t)(hi - lo), (off_t)(offset + lo));
      if (r < 0) {
        if (errno == EINTR) continue;
        err[t] = errno;
        return;
      }
      if (r == 0) return;
      lo += r;
      got[t] += r;
    }
  };
  std::vector<std::thread> th;
  for (int t = 1; t < threads; ++t) th.emplace_back(work, t);
  work(0);
  for (auto& x : th) x.join();
  ::close(fd);
  long long total = 0;
  for (int t = 0; t < threads; ++t) {
    if (err[t]) return -err[t];
    total += got[t];
  }
  return total;
}

HAPI long long mmj_file_size(const char* path) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return -1;
  std::fseek(f, 0, SEEK_END);
  long long n = std::ftell(f);
  std::fclose(f);
  return n;
}

// ---- CSV float packing -----------------------------------------------------------------------
// Formats n floats as comma-separated shortest round-trip decimals. Returns the length written
// (excluding the terminator), or the required capacity as a negative number if `cap` is too small.
HAPI long long mmj_pack_csv_f32(const float* x, long long n, char* out, long long cap) {
  std::string s;
  s.reserve((size_t)n * 12);
  char buf[64];
  for (long long i = 0; i < n; ++i) {
    int len = std::snprintf(buf, sizeof buf, "%.9g", (double)x[i]);
    // keep integral values readable as floats ("1" -> "1.0") like the reference's String(Float32)
    bool plain = true;
    for (int k = 0; k < len; ++k)
      if (buf[k] == '.' || buf[k] == 'e' || buf[k] == 'n' || buf[k] == 'i') plain = false;
    s.append(buf, (size_t)len);
    if (plain) s.append(".0");
    if (i + 1 < n) s.push_back(',');
  }
  if ((long long)s.size() + 1 > cap) return -((long long)s.size() + 1);
  std::memcpy(out, s.data(), s.size());
  out[s.size()] = 0;
  return (long long)s.size();
}

// Parses comma-separated decimals; unparsable fields become 0 (reference behaviour). Returns count.
HAPI long long mmj_unpack_csv_f32(const char* s, long long len, float* out, long long cap) {
  long long n = 0, i = 0;
  while (i < len) {
    long long j = i;
    while (j < len && s[j] != ',') ++j;
    if (j > i) {
      std::string field(s + i, (size_t)(j - i));
      char* end = nullptr;
      float v = std::strtof(field.c_str(), &end);
      if (end == field.c_str()) v = 0.f;
      if (n < cap) out[n] = v;
      ++n;
    }
    i = j + 1;
  }
  return n;
}

// ---- shuffles / hashing ------------------------------------------------------------------------
HAPI void mmj_lcg_shuffle(long long* idx, long long n, unsigned int seed) {
  for (long long i = 0; i < n; ++i) idx[i] = i;
  uint32_t state = seed;
  for (long long i = n - 1; i > 0; --i) {
    state = state * 1664525u + 1013904223u;
    long long j = (long long)(state % (uint32_t)(i + 1));
    long long t = idx[i];
    idx[i] = idx[j];
    idx[j] = t;
  }
}

HAPI unsigned long long mmj_fnv1a64(const unsigned char* data, long long n) {
  uint64_t h = 1469598103934665603ull;
  for (long long i = 0; i < n; ++i) {
    h ^= data[i];
    h *= 1099511628211ull;
  }
  return h;
}

// ---- vision CPU restatements -----------------------------------------------------------------
// Nearest-neighbour resize of an HWC u8 image: src index = (dst * src_size) / dst_size.
HAPI void mmj_cpu_resize_nearest_u8(const unsigned char* src, int H, int W, int C, unsigned char* dst,
                                    int OH, int OW) {
  for (int y = 0; y < OH; ++y) {
    int sy = (int)(((long long)y * H) / OH);
    if (sy >= H) sy = H - 1;
    for (int x = 0; x < OW; ++x) {
      int sx = (int)(((long long)x * W) / OW);
      if (sx >= W) sx = W - 1;
      const unsigned char* s = src + ((size_t)sy * W + sx) * C;
      unsigned char* d = dst + ((size_t)y * OW + x) * C;
      for (int c = 0; c < C; ++c) d[c] = s[c];
    }
  }
}

// gray = (299 R + 587 G + 114 B) / 1000 (integer arithmetic).
HAPI void mmj_cpu_rgb_to_gray_u8(const unsigned char* src, long long npix, unsigned char* dst) {
  for (long long i = 0; i < npix; ++i) {
    const unsigned char* p = src + i * 3;
    dst[i] = (unsigned char)((299 * p[0] + 587 * p[1] + 114 * p[2]) / 1000);
  }
}

// Bilinear resize (half-pixel centres, clamped), HWC u8.
HAPI void mmj_cpu_resize_bilinear_u8(const unsigned char* src, int H, int W, int C, unsigned char* dst,
                                     int OH, int OW) {
  const float sy = (float)H / OH, sx = (float)W / OW;
  for (int y = 0; y < OH; ++y) {
    float fy = (y + 0.5f) * sy - 0.5f;
    if (fy < 0) fy = 0;
    int y0 = (int)fy, y1 = y0 + 1 < H ? y0 + 1 : H - 1;
    float wy = fy - y0;
    for (int x = 0; x < OW; ++x) {
      float fx = (x + 0.5f) * sx - 0.5f;
      if (fx < 0) fx = 0;
      int x0 = (int)fx, x1 = x0 + 1 < W ? x0 + 1 : W - 1;
      float wx = fx - x0;
      for (int c = 0; c < C; ++c) {
        float a = src[((size_t)y0 * W + x0) * C + c], b = src[((size_t)y0 * W + x1) * C + c];
        float d = src[((size_t)y1 * W + x0) * C + c], e = src[((size_t)y1 * W + x1) * C + c];
        float v = (a * (1 - wx) + b * wx) * (1 - wy) + (d * (1 - wx) + e * wx) * wy;
        int iv = (int)(v + 0.5f);
        dst[((size_t)y * OW + x) * C + c] = (unsigned char)(iv < 0 ? 0 : (iv > 255 ? 255 : iv));
      }
    }
  }
}
