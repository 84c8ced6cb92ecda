// Breadth-first search by dynamic work creation: every round expands the
// frontier's edges with expt::lbs_workcreate (upsweep: claim unvisited
// neighbours and count their edges; downsweep: write the next frontier's
// segment starts and edge pointers), the way the reference's demo/bfs2.cu:23-65
// uses the engine. The graph is synthetic (seeded): random edges plus a long
// path, so that there are both wide and many levels. Levels are compared with
// a host breadth-first search; each round's segment array is checked to be the
// exclusive scan of the claimed vertices' degrees.
// Built by __graft_entry__.build(); the same source builds against the
// reference's headers (oracle/Makefile, target `ref`). Prints one line per
// check and "ALL PASSED" / "FAILED <n>".
#include <moderngpu/kernel_scan.hxx>
#include <moderngpu/kernel_workcreate.hxx>
#include <queue>
#include <random>

using namespace mgpu;

static int failures = 0;
static void report(const char* name, bool ok) {
  printf("%-52s %s\n", name, ok ? "ok" : "FAIL");
  if(!ok) ++failures;
}

struct frontier_t {
  int count;                  // edges leaving the frontier
  int num_segments;           // vertices in the frontier
  mem_t<int> segments;        // exclusive scan of their degrees
  mem_t<int> edge_indices;    // where each one's adjacency list starts
};

static bool run_graph(int num_vertices, int random_edges, int path_length,
  int seed, context_t& context) {
  // Build an undirected graph in CSR form on the host.
  std::mt19937 rng(seed);
  std::uniform_int_distribution<int> pick(0, num_vertices - 1);
  std::vector<std::pair<int, int> > pairs;
  for(int e = 0; e < random_edges; ++e) {
    int u = pick(rng), v = pick(rng);
    if(u != v) { pairs.push_back({ u, v }); pairs.push_back({ v, u }); }
  }
  for(int i = 0; i + 1 < path_length; ++i) {
    pairs.push_back({ i, i + 1 });
    pairs.push_back({ i + 1, i });
  }
  std::sort(pairs.begin(), pairs.end());
  std::vector<int> offsets(num_vertices + 1, 0), edges(pairs.size());
  for(size_t e = 0; e < pairs.size(); ++e) {
    ++offsets[pairs[e].first + 1];
    edges[e] = pairs[e].second;
  }
  for(int v = 0; v < num_vertices; ++v) offsets[v + 1] += offsets[v];

  // Host levels.
  std::vector<int> want(num_vertices, -1);
  std::queue<int> queue;
  want[0] = 0;
  queue.push(0);
  while(!queue.empty()) {
    int u = queue.front(); queue.pop();
    for(int e = offsets[u]; e < offsets[u + 1]; ++e)
      if(-1 == want[edges[e]]) { want[edges[e]] = want[u] + 1; queue.push(edges[e]); }
  }

  mem_t<int> offsets_device = to_mem(offsets, context);
  mem_t<int> edges_device = to_mem(edges, context);
  const int* vertices = offsets_device.data();
  const int* edge_list = edges_device.data();
  std::vector<int> initial(num_vertices, -1);
  initial[0] = 0;
  mem_t<int> values_device = to_mem(initial, context);
  int* values = values_device.data();

  frontier_t wl;
  wl.count = offsets[1] - offsets[0];
  wl.num_segments = 1;
  wl.segments = to_mem(std::vector<int>(1, 0), context);
  wl.edge_indices = to_mem(std::vector<int>(1, offsets[0]), context);

  bool ok = true;
  for(int cur = 0; wl.num_segments && ok; ++cur) {
    auto engine = expt::lbs_workcreate(wl.count, wl.segments.data(),
      wl.num_segments, context);
    auto next = engine.upsweep(
      [=]MGPU_DEVICE(int index, int seg, int rank, tuple<int> desc) {
        int neighbor = edge_list[get<0>(desc) + rank];
        int created = 0;
        if(-1 == atomicCAS(values + neighbor, -1, cur + 1))
          created = vertices[neighbor + 1] - vertices[neighbor];
        return created;
      }, make_tuple(wl.edge_indices.data()));

    mem_t<int> edge_indices(next.num_segments, context);
    mem_t<int> vertex_of(next.num_segments, context);
    mem_t<int> segments = engine.downsweep(
      [=]MGPU_DEVICE(int dest_seg, int index, int seg, int rank,
        tuple<int> desc, int* out_edge_indices, int* out_vertex) {
        int neighbor = edge_list[get<0>(desc) + rank];
        int begin = vertices[neighbor], end = vertices[neighbor + 1];
        out_edge_indices[dest_seg] = begin;
        out_vertex[dest_seg] = neighbor;
        return end - begin;
      }, make_tuple(wl.edge_indices.data()), edge_indices.data(),
      vertex_of.data());

    // The new segment array is the exclusive scan of the degrees of the
    // vertices just claimed (in the order the engine compacted them), and
    // its total is the count the upsweep returned.
    std::vector<int> seg_host = from_mem(segments);
    std::vector<int> vertex_host = from_mem(vertex_of);
    std::vector<int> edge_host = from_mem(edge_indices);
    int running = 0;
    for(int j = 0; j < next.num_segments && ok; ++j) {
      int v = vertex_host[j];
      ok = seg_host[j] == running && edge_host[j] == offsets[v] &&
        want[v] == cur + 1 && offsets[v + 1] > offsets[v];
      running += offsets[v + 1] - offsets[v];
    }
    ok = ok && running == next.count;

    wl.count = next.count;
    wl.num_segments = next.num_segments;
    wl.segments = std::move(segments);
    wl.edge_indices = std::move(edge_indices);
  }
  std::vector<int> got = from_mem(values_device);
  return ok && got == want;
}

int main() {
  standard_context_t context(false);
  report("bfs, 200,000 vertices, 800,000 random edges",
    run_graph(200000, 800000, 2, 1, context));
  report("bfs, sparse graph with a 3,000-vertex path",
    run_graph(50000, 20000, 3000, 2, context));
  report("bfs, dense small graph",
    run_graph(2000, 400000, 2, 3, context));
  report("bfs, source without edges",
    run_graph(10, 0, 1, 4, context));
  context.synchronize();
  if(failures) printf("FAILED %d\n", failures);
  else printf("ALL PASSED\n");
  return failures;
}
