// Builds EmbeddingBag_TRT plugins through the host driver, serialises them, and feeds damaged
// copies of the blobs (truncations, byte flips, inflated size fields, layout-"002" headers)
// back through the creator's deserializePlugin.  Built by tests/test_sanitizers.py with
// AddressSanitizer and UndefinedBehaviorSanitizer; no GPU is needed (nothing is enqueued).
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

struct fwd_eb_host;
extern "C" {
fwd_eb_host* fwd_eb_host_build(const void* table, int half_table, int count, int dim, int offset, int op,
                               long long padding_idx, int include_last_offset, int half_output,
                               int idx_rank, const int* idx_dims, int off_rank, const int* off_dims,
                               int weights_rank, const int* weights_dims);
void fwd_eb_host_free(fwd_eb_host* h);
size_t fwd_eb_host_blob(fwd_eb_host* h, void* dst, size_t cap);
fwd_eb_host* fwd_eb_host_load(const void* blob, size_t len, const fwd_eb_host* like);
fwd_eb_host* fwd_eb_host_clone_context(const fwd_eb_host* src);
}

int main() {
  std::mt19937 rng(11);
  int loaded = 0, refused = 0;
  for (int variant = 0; variant < 3; ++variant) {
    const int half = variant == 1, count = 9 + variant, dim = 6 + 2 * variant;
    std::vector<float> table((size_t)count * dim);
    for (auto& v : table) v = (float)(rng() % 1000) / 100.0f;
    const int idx_dims[1] = {40}, off_dims[1] = {5}, w_dims[1] = {40};
    const int op = variant == 0 ? 2 : (variant == 1 ? 1 : 0);   // max; mean over fp16; weighted sum
    fwd_eb_host* h = fwd_eb_host_build(table.data(), half, count, dim, 3, op, variant == 2 ? 4 : -1,
                                       variant == 2, half, 1, idx_dims, 1, off_dims, variant == 2 ? 1 : 0, w_dims);
    if (!h) return 2;
    std::vector<unsigned char> blob(fwd_eb_host_blob(h, nullptr, 0));
    fwd_eb_host_blob(h, blob.data(), blob.size());
    if (blob.empty()) return 3;
    auto attempt = [&](const std::vector<unsigned char>& b) {
      // an exact-size heap copy: reading one byte past the blob is an error the sanitizer sees
      std::vector<unsigned char> exact(b.begin(), b.end());
      fwd_eb_host* g = fwd_eb_host_load(exact.data(), exact.size(), h);
      if (g) {
        ++loaded;
        if (fwd_eb_host* c = fwd_eb_host_clone_context(g)) fwd_eb_host_free(c);
        fwd_eb_host_free(g);
      } else {
        ++refused;
      }
    };
    attempt(blob);
    for (size_t n = 0; n < blob.size(); n += 3) attempt(std::vector<unsigned char>(blob.begin(), blob.begin() + n));
    for (int k = 0; k < 400; ++k) {
      std::vector<unsigned char> b = blob;
      const int flips = 1 + (int)(rng() % 4);
      for (int f = 0; f < flips; ++f) b[rng() % b.size()] = (unsigned char)(rng() & 0xff);
      attempt(b);
    }
    for (int k = 0; k < 60; ++k) {   // the header's sizes: dim, count, data_offset, op, element count
      std::vector<unsigned char> b = blob;
      const size_t field = (rng() % 5) * 4;
      const int64_t values[] = {0, -1, 1, 0x7fffffff, (int64_t)0x80000000u, 1 << 20, -2};
      const int64_t v = values[rng() % 7];
      std::memcpy(b.data() + field, &v, field == 16 ? 8 : 4);
      attempt(b);
    }
    for (int k = 0; k < 60; ++k) {   // something that claims to be the external-weights layout
      std::vector<unsigned char> b(4 + 3 + 4 + 8 + 8 + 4 + 4 + 8 + 4 + (rng() % 40));
      for (auto& c : b) c = (unsigned char)(rng() & 0xff);
      const int32_t marker = -2;
      std::memcpy(b.data(), &marker, 4);
      std::memcpy(b.data() + 4, "002", 3);
      attempt(b);
    }
    fwd_eb_host_free(h);
  }
  std::printf("loaded %d refused %d\n", loaded, refused);
  return (loaded > 0 && refused > 0) ? 0 : 4;
}
