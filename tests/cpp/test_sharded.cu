// mgpu::sharded_segreduce, the C++ entry of the multi-GPU layer: one array
// with ONE global table of 64-bit segment starts is cut on the devices into
// shards (shard-local int32 tables by lower bound at every shard edge), every
// shard is reduced by the single-GPU kernel, and the segments that straddle
// shard edges are completed through boundary records that travel between the
// GPUs' mailboxes. The assembled result must equal the host loop of the
// reference's test (tests/test_segreduce.cu:40-49) over the WHOLE array: bit
// for bit for integers and max, within 1e-12 for fp64 sums.
//
// Runs on every GPU of the machine (up to four), two shards per GPU; with one
// GPU the same chain of records runs through that GPU's own mailbox. 70 steps
// per case, so that the 64-slot rings of the mailboxes wrap.
// Built by __graft_entry__.build(). Prints one line per check and
// "ALL PASSED" / "FAILED <n>".
#include <moderngpu/kernel_sharded.hxx>
#include <random>
#include <cmath>

using namespace mgpu;

static int failures = 0;
static void report(const char* name, bool ok) {
  printf("%-64s %s\n", name, ok ? "ok" : "FAIL");
  if(!ok) ++failures;
}

// Segment starts of three shapes: log-normal lengths (many segments straddle
// shard edges), a few very long segments (a shard may hold no start at all),
// and one segment.
static std::vector<long long> make_segments(int kind, long long count,
  std::mt19937& rng) {
  std::vector<long long> seg;
  if(0 == kind) {
    std::normal_distribution<double> z(0.0, 1.0);
    long long at = 0;
    while(at <= count) {
      seg.push_back(at);
      at += (long long)std::floor(std::exp(3.0 + 1.5 * z(rng)));
    }
    seg.push_back(count);        // trailing empty segments at the array's end
    seg.push_back(count);
  } else if(1 == kind) {
    seg = { 0, 10, 11, count - count / 40 };
  } else {
    seg = { 0 };
  }
  return seg;
}

template<typename type_t, typename op_t>
static bool run_case(shard_group_t& group, int kind, long long count,
  op_t op, type_t init, bool exact, int steps) {
  std::mt19937 rng(41 + kind);
  std::vector<long long> seg = make_segments(kind, count, rng);
  const long long num_segments = (long long)seg.size();
  std::vector<type_t> values((size_t)count);
  for(auto& v : values) {
    if(std::is_integral<type_t>::value) v = (type_t)((int)(rng() % 2001) - 1000);
    else v = (type_t)(((double)(rng() % 2000001) - 1e6));
  }

  // Host loop over the whole array.
  std::vector<type_t> want((size_t)num_segments);
  std::vector<double> scale((size_t)num_segments, 0.0);
  for(long long s = 0; s < num_segments; ++s) {
    long long begin = seg[s], end = s + 1 < num_segments ? seg[s + 1] : count;
    type_t x = init;
    long double wide = 0, mag = 0;
    for(long long i = begin; i < end; ++i) {
      x = (i == begin) ? values[i] : op(x, values[i]);
      wide += (long double)values[i];
      mag += std::fabs((long double)values[i]);
    }
    want[s] = x;
    if(!exact && end > begin) { want[s] = (type_t)wide; scale[s] = (double)mag; }
  }

  // The global table lives on the first GPU; the others read it from there.
  const int shards = group.num_shards();
  cudaSetDevice(group.device_of(0));
  long long* seg_device = nullptr;
  cudaMalloc((void**)&seg_device, sizeof(long long) * num_segments);
  cudaMemcpy(seg_device, seg.data(), sizeof(long long) * num_segments,
    cudaMemcpyHostToDevice);
  shard_plan_t plan = sharded_partition(seg_device, num_segments, count, group);

  std::vector<type_t*> inputs(shards), outputs(shards);
  long long covered = 0;
  bool ok = true;
  for(int v = 0; v < shards; ++v) {
    cudaSetDevice(group.device_of(v));
    cudaMalloc((void**)&inputs[v], sizeof(type_t) * (size_t)(plan.items(v) + 1));
    cudaMalloc((void**)&outputs[v], sizeof(type_t) * (size_t)plan.outputs(v));
    cudaMemcpy(inputs[v], values.data() + plan.item_begin[v],
      sizeof(type_t) * (size_t)plan.items(v), cudaMemcpyHostToDevice);
    ok = ok && plan.first_segment[v] == covered;
    covered += plan.outputs(v) - 1;
  }
  ok = ok && covered == num_segments;

  for(int step = 0; step < steps; ++step)
    sharded_segreduce((const type_t* const*)inputs.data(), plan,
      outputs.data(), op, init, group);
  try {
    group.synchronize();
  } catch(cuda_exception_t& e) {
    printf("  synchronize: %s\n", e.what());
    ok = false;
  }

  for(int v = 0; v < shards; ++v) {
    cudaSetDevice(group.device_of(v));
    std::vector<type_t> got((size_t)plan.outputs(v));
    cudaMemcpy(got.data(), outputs[v], sizeof(type_t) * got.size(),
      cudaMemcpyDeviceToHost);
    for(int j = 1; j < plan.outputs(v); ++j) {
      long long s = plan.first_segment[v] + j - 1;
      bool same = exact ? got[j] == want[s] :
        std::fabs((double)got[j] - (double)want[s]) <=
          1e-12 * std::max(std::fabs((double)want[s]), scale[s]);
      if(!same && ok) {
        printf("  shard %d segment %lld: got %.17g want %.17g\n", v, s,
          (double)got[j], (double)want[s]);
        ok = false;
      }
    }
    cudaFree(inputs[v]);
    cudaFree(outputs[v]);
  }
  cudaSetDevice(group.device_of(0));
  cudaFree(seg_device);
  return ok;
}

int main(int argc, char** argv) {
  int available = 0;
  cudaGetDeviceCount(&available);
  if(!available) { printf("no GPU\n"); return 2; }
  int gpus = available < 4 ? available : 4;
  if(argc > 1) gpus = std::min(gpus, std::max(1, atoi(argv[1])));
  std::vector<int> devices;
  for(int g = 0; g < gpus; ++g) devices.push_back(g);
  printf("%d GPU(s), 2 shards each\n", gpus);

  const long long count = 6000011;
  const int steps = 70;
  {
    shard_group_t group(devices, 2);
    report("int64 plus, log-normal segments",
      run_case<long long>(group, 0, count, plus_t<long long>(), -7ll, true, steps));
    report("fp64 max, log-normal segments",
      run_case<double>(group, 0, count, maximum_t<double>(), -7.0, true, steps));
    report("fp64 plus, log-normal segments (1e-12)",
      run_case<double>(group, 0, count, plus_t<double>(), -7.0, false, steps));
    report("int32 plus, four segments (shards without a start)",
      run_case<int>(group, 1, count, plus_t<int>(), -1, true, steps));
    report("fp32 min, one segment over every shard",
      run_case<float>(group, 2, count, minimum_t<float>(), 0.0f, true, steps));
  }
  {
    // One shard per GPU and an array of a size no shard divides evenly.
    shard_group_t group(devices, 1);
    report("int32 max, one shard per GPU",
      run_case<int>(group, 0, 1000003, maximum_t<int>(), -5, true, 3));
  }
  if(failures) printf("FAILED %d\n", failures);
  else printf("ALL PASSED\n");
  return failures ? 1 : 0;
}
