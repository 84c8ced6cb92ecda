// Golden-vector generator: runs the REFERENCE's own host-callable
// merge_path<bounds_upper> (src/moderngpu/cta_merge.hxx:8-29, used by
// load_balance_partitions, src/moderngpu/search.hxx:29-37) on the CPU and
// writes tests/golden/lbs_partitions.json. Segment offsets are generated the
// way the reference's tests do (tests/test_segreduce.cu:16-22 with
// std::mt19937, tests/test_load_balance.cu:11-16 uniform spacing).
//
// Built and run only where the reference checkout is present:
//   make -C oracle ref && oracle/_ref/ref_host_golden tests/golden/lbs_partitions.json
// Test infrastructure; nothing in the shipped library uses it.
#include <moderngpu/cta_merge.hxx>
#include <moderngpu/operators.hxx>
#include <algorithm>
#include <cstdio>
#include <random>
#include <vector>

using namespace mgpu;

static std::vector<int> random_segments(int count, int num_segments, int seed) {
  std::mt19937 mt19937(seed);
  std::uniform_int_distribution<int> dist(0, count);
  std::vector<int> s(num_segments);
  s[0] = 0;
  for(int i = 1; i < num_segments; ++i) s[i] = dist(mt19937);
  std::sort(s.begin() + 1, s.end());
  return s;
}

static void emit_case(FILE* f, const char* name, int count,
  const std::vector<int>& seg, const std::vector<int>& spacings, bool last) {
  int ns = (int)seg.size();
  fprintf(f, "  {\"name\": \"%s\", \"count\": %d, \"segments\": [", name, count);
  for(int i = 0; i < ns; ++i) fprintf(f, "%s%d", i ? "," : "", seg[i]);
  fprintf(f, "], \"partitions\": {");
  for(size_t k = 0; k < spacings.size(); ++k) {
    int spacing = spacings[k];
    int total = count + ns;
    int n = (total + spacing - 1) / spacing + 1;
    fprintf(f, "%s\"%d\": [", k ? ", " : "", spacing);
    for(int p = 0; p < n; ++p) {
      int diag = std::min(spacing * p, total);
      int mp = merge_path<bounds_upper>(counting_iterator_t<int>(0), count,
        seg.data(), ns, diag, less_t<int>());
      fprintf(f, "%s%d", p ? "," : "", mp);
    }
    fprintf(f, "]");
  }
  fprintf(f, "}}%s\n", last ? "" : ",");
}

int main(int argc, char** argv) {
  const char* path = argc > 1 ? argv[1] : "lbs_partitions.json";
  FILE* f = fopen(path, "w");
  if(!f) { perror(path); return 1; }
  fprintf(f, "{\"generator\": \"oracle/ref_host_golden.cu\", \"cases\": [\n");
  emit_case(f, "random_1000_10_seed0", 1000, random_segments(1000, 10, 0), {1, 7, 896}, false);
  emit_case(f, "random_1000_10_seed1", 1000, random_segments(1000, 10, 1), {1, 7, 896}, false);
  emit_case(f, "random_1000_37_seed2", 1000, random_segments(1000, 37, 2), {1, 13, 128}, false);
  emit_case(f, "many_empty_50_200_seed3", 50, random_segments(50, 200, 3), {1, 16}, false);
  {
    int count = 2030, spacing = 100;
    std::vector<int> s((count + spacing - 1) / spacing);
    for(size_t i = 0; i < s.size(); ++i) s[i] = (int)i * spacing;
    emit_case(f, "uniform_2030_by_100", count, s, {1, 128}, false);
  }
  emit_case(f, "no_items_0_5", 0, std::vector<int>(5, 0), {1, 4}, false);
  emit_case(f, "random_100000_1000_seed5", 100000, random_segments(100000, 1000, 5), {896, 7160}, true);
  fprintf(f, "]}\n");
  fclose(f);
  return 0;
}
