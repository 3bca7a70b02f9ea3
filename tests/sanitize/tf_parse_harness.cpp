// Parses every GraphDef file named on the command line (argv[1] = comma-separated output names)
// through the same entry point the TensorFlow parser slice exports, reads back every description
// it found, and frees it.  Built by tests/test_sanitizers.py with AddressSanitizer and
// UndefinedBehaviorSanitizer: a wild read, an overflow or a leak in the GraphDef reader or in
// the pattern matcher ends the process with a non-zero status.
#include <cstddef>
#include <cstdio>
#include <vector>

struct fwd_eb_tf_parsed;
extern "C" {
fwd_eb_tf_parsed* fwd_eb_tf_parse(const char* path, const char* outputs, char* err, size_t err_cap);
void fwd_eb_tf_free(fwd_eb_tf_parsed* p);
int fwd_eb_tf_num_descs(const fwd_eb_tf_parsed* p);
const char* fwd_eb_tf_desc_node(const fwd_eb_tf_parsed* p, int i);
const char* fwd_eb_tf_desc_input(const fwd_eb_tf_parsed* p, int i);
int fwd_eb_tf_desc_info(const fwd_eb_tf_parsed* p, int i, int* dim, int* count, int* offset, int* op,
                        int* half_table);
size_t fwd_eb_tf_desc_weights(const fwd_eb_tf_parsed* p, int i, void* dst, size_t cap);
}

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  int parsed = 0, refused = 0;
  for (int a = 2; a < argc; ++a) {
    char err[256] = "";
    fwd_eb_tf_parsed* p = fwd_eb_tf_parse(argv[a], argv[1], err, sizeof(err));
    if (!p) {
      ++refused;
      if (!err[0]) return 3;  // a refusal always says why
      continue;
    }
    ++parsed;
    const int n = fwd_eb_tf_num_descs(p);
    for (int i = 0; i < n; ++i) {
      int dim = 0, count = 0, offset = 0, op = 0, half = 0;
      if (fwd_eb_tf_desc_info(p, i, &dim, &count, &offset, &op, &half) != 0) return 4;
      (void)fwd_eb_tf_desc_node(p, i);
      (void)fwd_eb_tf_desc_input(p, i);
      const size_t bytes = fwd_eb_tf_desc_weights(p, i, nullptr, 0);
      std::vector<char> w(bytes);
      if (fwd_eb_tf_desc_weights(p, i, w.data(), w.size()) != bytes) return 5;
      if (bytes != (size_t)dim * (size_t)count * (half ? 2u : 4u)) return 6;
    }
    fwd_eb_tf_free(p);
  }
  std::printf("parsed %d refused %d\n", parsed, refused);
  return 0;
}
