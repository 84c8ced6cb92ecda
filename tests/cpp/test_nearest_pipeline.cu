// Integration test of the whole call chain a user of the library strings
// together, in the shape of the reference's demo/cities.cu:143-236 ("for every
// city, the closest other cities of its state"):
//
//   scan -> interval_expand -> transform_lbs (cached tuple) -> scan in place
//        -> lbs_segreduce<launch_params_t<128, 3>> with a 24-byte value type,
//           a user-written merge operator and a two-pointer cached tuple.
//
// The data is synthetic (seeded): groups of points on an integer grid, so
// that squared distances are exact in float and the result can be compared
// bit for bit with a brute-force host loop. The final segmented sort of the
// demo is outside this library's scope and is left out.
// Built by __graft_entry__.build() into tests/cpp/build/; the same source
// builds against the reference's headers (oracle/Makefile, target `ref`).
// Prints one line per check and "ALL PASSED" / "FAILED <n>"; exit code = the
// number of failed checks.
#include <moderngpu/kernel_intervalmove.hxx>
#include <moderngpu/kernel_load_balance.hxx>
#include <moderngpu/kernel_scan.hxx>
#include <moderngpu/kernel_segreduce.hxx>
#include <cfloat>
#include <random>

using namespace mgpu;

static int failures = 0;
static void report(const char* name, bool ok) {
  printf("%-52s %s\n", name, ok ? "ok" : "FAIL");
  if(!ok) ++failures;
}

enum { nearest_count = 3 };

// The `nearest_count` best (score, point) pairs seen so far, best first.
struct nearest_t {
  float score[nearest_count];
  int point[nearest_count];
};

MGPU_HOST_DEVICE bool before(float sa, int pa, float sb, int pb) {
  return sa < sb || (sa == sb && pa < pb);
}

// Merge of two sorted lists, cut to nearest_count entries. Ties are broken by
// the point index, so the operator is commutative as well as associative and
// the result does not depend on the order of evaluation.
struct merge_nearest_t {
  MGPU_HOST_DEVICE nearest_t operator()(nearest_t a, nearest_t b) const {
    nearest_t c;
    int i = 0, j = 0;
    for(int k = 0; k < nearest_count; ++k) {
      bool from_a = !before(b.score[j], b.point[j], a.score[i], a.point[i]);
      c.score[k] = from_a ? a.score[i] : b.score[j];
      c.point[k] = from_a ? a.point[i] : b.point[j];
      if(from_a) ++i; else ++j;
    }
    return c;
  }
};

MGPU_HOST_DEVICE nearest_t single(float score, int point) {
  nearest_t x;
  for(int k = 0; k < nearest_count; ++k) { x.score[k] = FLT_MAX; x.point[k] = -1; }
  x.score[0] = score;
  x.point[0] = point;
  return x;
}

MGPU_HOST_DEVICE float squared_distance(int2 a, int2 b) {
  float dx = (float)(a.x - b.x), dy = (float)(a.y - b.y);
  return dx * dx + dy * dy;
}

static bool same(const nearest_t& a, const nearest_t& b) {
  for(int k = 0; k < nearest_count; ++k)
    if(a.score[k] != b.score[k] || a.point[k] != b.point[k]) return false;
  return true;
}

static void run_case(const char* label, const std::vector<int>& group_sizes,
  int seed, context_t& context) {
  const int num_groups = (int)group_sizes.size();
  int num_points = 0;
  long long num_pairs_wide = 0;
  for(int n : group_sizes) {
    num_points += n;
    num_pairs_wide += (long long)n * (n > 0 ? n - 1 : 0);
  }
  const int num_pairs = (int)num_pairs_wide;

  std::mt19937 rng(seed);
  std::uniform_int_distribution<int> coord(0, 2000);
  std::vector<int2> position(num_points);
  for(int2& p : position) p = make_int2(coord(rng), coord(rng));

  mem_t<int> sizes_device = to_mem(group_sizes, context);
  mem_t<int2> position_device = to_mem(position, context);
  const int* sizes_data = sizes_device.data();
  const int2* position_data = position_device.data();

  // 1. Group sizes -> group start offsets.
  mem_t<int> group_start(num_groups, context);
  scan(sizes_data, num_groups, group_start.data(), context);

  // 2. For every point, the first point of its group.
  mem_t<int> first_of_group(num_points, context);
  interval_expand(group_start.data(), num_points, group_start.data(),
    num_groups, first_of_group.data(), context);

  // 3. For every point, how many other points its group holds.
  mem_t<int> pair_start(num_points, context);
  int* pair_start_data = pair_start.data();
  transform_lbs([=]MGPU_DEVICE(int index, int seg, int rank,
    tuple<int> group_size) {
    pair_start_data[index] = get<0>(group_size) - 1;
  }, num_points, group_start.data(), num_groups, make_tuple(sizes_data),
    context);

  // 4. ... turned into the start offsets of each point's run of pairs.
  scan(pair_start.data(), num_points, pair_start.data(), context);

  // 5. One work item per ordered pair of distinct points of a group; the
  // segmented reduction keeps each point's nearest_count closest partners.
  auto score = [=]MGPU_DEVICE(int index, int point_i, int rank,
    tuple<int, int2> cached) {
    int point_j = get<0>(cached) + rank;
    if(point_j >= point_i) ++point_j;          // skip the point itself
    return single(squared_distance(get<1>(cached), position_data[point_j]),
      point_j);
  };
  nearest_t init = single(0, -1);
  for(int k = 0; k < nearest_count; ++k) { init.score[k] = 0; init.point[k] = -1; }
  mem_t<nearest_t> nearest(num_points, context);
  lbs_segreduce<launch_params_t<128, 3> >(score, num_pairs, pair_start.data(),
    num_points, make_tuple(first_of_group.data(), position_data),
    nearest.data(), merge_nearest_t(), init, context);

  std::vector<int> group_start_host = from_mem(group_start);
  std::vector<int> first_host = from_mem(first_of_group);
  std::vector<int> pair_start_host = from_mem(pair_start);
  std::vector<nearest_t> nearest_host = from_mem(nearest);

  // Host loops.
  bool ok_start = true, ok_first = true, ok_pairs = true, ok_nearest = true;
  int point = 0, pairs = 0;
  for(int g = 0; g < num_groups; ++g) {
    ok_start &= group_start_host[g] == point;
    const int n = group_sizes[g], first = point;
    for(int i = first; i < first + n; ++i, ++point) {
      ok_first &= first_host[i] == first;
      ok_pairs &= pair_start_host[i] == pairs;
      pairs += n - 1;
      nearest_t want = init;
      bool any = false;
      for(int j = first; j < first + n; ++j) {
        if(j == i) continue;
        nearest_t x = single(squared_distance(position[i], position[j]), j);
        want = any ? merge_nearest_t()(want, x) : x;
        any = true;
      }
      ok_nearest &= same(want, nearest_host[i]);
    }
  }
  char name[128];
  snprintf(name, sizeof(name), "%s: scan of group sizes", label);
  report(name, ok_start);
  snprintf(name, sizeof(name), "%s: interval_expand", label);
  report(name, ok_first);
  snprintf(name, sizeof(name), "%s: transform_lbs + scan in place", label);
  report(name, ok_pairs && pairs == num_pairs);
  snprintf(name, sizeof(name), "%s: lbs_segreduce, %d pairs", label, num_pairs);
  report(name, ok_nearest);
}

int main() {
  standard_context_t context(false);

  {
    // Many groups of uneven size, some empty, some with a single point (whose
    // run of pairs is empty: the result must be `init`).
    std::mt19937 rng(5);
    std::uniform_int_distribution<int> size(0, 120);
    std::vector<int> sizes(3000);
    for(int& n : sizes) n = size(rng);
    sizes[0] = 1; sizes[7] = 0; sizes[8] = 0; sizes[2999] = 1;
    run_case("uneven groups", sizes, 11, context);
  }
  {
    // A few large groups: each point's run spans many items, a group's runs
    // span many tiles.
    std::vector<int> sizes = { 1500, 2, 0, 900, 1, 1200 };
    run_case("large groups", sizes, 12, context);
  }
  {
    std::vector<int> sizes = { 2 };
    run_case("two points", sizes, 13, context);
  }

  context.synchronize();
  if(failures) printf("FAILED %d\n", failures);
  else printf("ALL PASSED\n");
  return failures;
}
