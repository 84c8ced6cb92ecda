// C entry points over the UNMODIFIED reference headers (moderngpu 2.x,
// included from the reference checkout where it lies; nothing is copied).
// Compiled for sm_100a into oracle/_ref/libmgpu_ref.so by oracle/Makefile.
//
// TEST INFRASTRUCTURE: used on a GPU (a) as a second oracle — the reference's
// own CUDA build run on the same inputs — and (b) as the "reference CUDA
// build" baseline that the benchmark reports. The shipped library never loads
// it. Every function takes device pointers, runs on the legacy default
// stream through the reference's stock standard_context_t, and returns 0 or a
// cudaError_t.
#include <moderngpu/kernel_segreduce.hxx>
#include <moderngpu/kernel_load_balance.hxx>
#include <moderngpu/kernel_intervalmove.hxx>
#include <map>

using namespace mgpu;

namespace {

standard_context_t& stock_context() {
  static standard_context_t context(false);
  return context;
}

// A context that recycles freed blocks, so the reference's kernels can be
// timed without its per-call cudaMalloc / cudaFree.
class pooled_context_t : public standard_context_t {
  std::multimap<size_t, void*> free_blocks;
  std::map<void*, size_t> sizes;
public:
  pooled_context_t() : standard_context_t(false) { }
  void* alloc(size_t size, memory_space_t space) override {
    if(memory_space_device != space || !size)
      return standard_context_t::alloc(size, space);
    auto it = free_blocks.lower_bound(size);
    if(it != free_blocks.end() && it->first <= 2 * size + 4096) {
      void* p = it->second;
      free_blocks.erase(it);
      return p;
    }
    void* p = standard_context_t::alloc(size, space);
    sizes[p] = size;
    return p;
  }
  void free(void* p, memory_space_t space) override {
    if(memory_space_device != space || !p) {
      standard_context_t::free(p, space);
      return;
    }
    free_blocks.insert(std::make_pair(sizes[p], p));
  }
};

pooled_context_t& pooled_context() {
  static pooled_context_t context;
  return context;
}

context_t& pick(int pooled) {
  if(pooled) return pooled_context();
  return stock_context();
}

int finish() {
  cudaError_t e = cudaDeviceSynchronize();
  if(cudaSuccess == e) e = cudaGetLastError();
  return (int)e;
}

template<typename type_t, typename op_t>
int run_segreduce(const type_t* input, int count, const int* segments,
  int num_segments, type_t* output, type_t init, int pooled, int sync) {
  try {
    segreduce(input, count, segments, num_segments, output, op_t(), init,
      pick(pooled));
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return sync ? finish() : 0;
}

} // namespace

extern "C" {

// op: 0 plus, 1 max, 2 min. pooled: 0 stock context, 1 pooled context.
#define REF_SEGREDUCE(NAME, T)                                                 \
int NAME(const T* input, int count, const int* segments, int num_segments,    \
  T* output, T init, int op, int pooled, int sync) {                          \
  if(0 == op) return run_segreduce<T, plus_t<T> >(input, count, segments,     \
    num_segments, output, init, pooled, sync);                                \
  if(1 == op) return run_segreduce<T, maximum_t<T> >(input, count, segments,  \
    num_segments, output, init, pooled, sync);                                \
  return run_segreduce<T, minimum_t<T> >(input, count, segments,              \
    num_segments, output, init, pooled, sync);                                \
}
REF_SEGREDUCE(ref_segreduce_f32, float)
REF_SEGREDUCE(ref_segreduce_f64, double)
REF_SEGREDUCE(ref_segreduce_i32, int)
REF_SEGREDUCE(ref_segreduce_i64, long long)

// The reference's own test workload (tests/test_segreduce.cu:31-35).
int ref_transform_segreduce_index_mod(int count, const int* segments,
  int num_segments, int* output, int init, int modulus) {
  try {
    transform_segreduce([=]MGPU_DEVICE(int index) { return index % modulus; },
      count, segments, num_segments, output, plus_t<int>(), init,
      stock_context());
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return finish();
}

int ref_spmv_f32(const float* matrix, const int* columns, const float* x,
  int nnz, const int* row_starts, int rows, float* y, int pooled, int sync) {
  try {
    spmv(matrix, columns, x, nnz, row_starts, rows, y, pick(pooled));
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return sync ? finish() : 0;
}

int ref_load_balance_search(int count, const int* segments, int num_segments,
  int* seg_out, int pooled, int sync) {
  try {
    load_balance_search(count, segments, num_segments, seg_out, pick(pooled));
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return sync ? finish() : 0;
}

// transform_lbs recording (seg, rank) per item.
int ref_lbs_seg_rank(int count, const int* segments, int num_segments,
  int* seg_out, int* rank_out, int pooled, int sync) {
  try {
    transform_lbs([=]MGPU_DEVICE(int index, int seg, int rank) {
      seg_out[index] = seg;
      rank_out[index] = rank;
    }, count, segments, num_segments, pick(pooled));
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return sync ? finish() : 0;
}

int ref_interval_expand_i32(const int* input, int count, const int* segments,
  int num_segments, int* output) {
  try {
    interval_expand(input, count, segments, num_segments, output,
      stock_context());
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return finish();
}

int ref_load_balance_partitions(int count, const int* segments,
  int num_segments, int spacing, int* partitions) {
  try {
    mem_t<int> mp = load_balance_partitions((int64_t)count, segments,
      num_segments, spacing, stock_context());
    cudaMemcpy(partitions, mp.data(), sizeof(int) * mp.size(),
      cudaMemcpyDeviceToDevice);
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return finish();
}

// lbs_segreduce of f(index, seg, rank) = seg + rank
// (tests/test_segreduce.cu:11-13,29-30).
int ref_lbs_segreduce_seg_plus_rank(int count, const int* segments,
  int num_segments, int* output, int init) {
  try {
    lbs_segreduce([]MGPU_DEVICE(int index, int seg, int rank) {
      return seg + rank;
    }, count, segments, num_segments, output, plus_t<int>(), init,
      stock_context());
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return finish();
}

// lbs_segreduce with a per-segment cached weight
// (src/moderngpu/kernel_segreduce.hxx:303-387):
// f(index, seg, rank, tuple<weight>) = values[index] * weight, op plus, init 0.
int ref_lbs_segreduce_weighted_f32(const float* values, int count,
  const int* segments, int num_segments, const float* weights, float* output,
  int pooled, int sync) {
  try {
    lbs_segreduce([=]MGPU_DEVICE(int index, int seg, int rank,
      tuple<float> weight) {
      return values[index] * get<0>(weight);
    }, count, segments, num_segments, make_tuple(weights), output,
      plus_t<float>(), 0.0f, pick(pooled));
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return sync ? finish() : 0;
}

// Host-vector round trip through the reference's API: to_mem, segreduce,
// from_mem (src/moderngpu/memory.hxx:61-75), fp32 plus.
int ref_segreduce_f32_host(const float* input_host, int count,
  const int* segments_host, int num_segments, float* output_host, float init) {
  try {
    context_t& context = stock_context();
    mem_t<float> input(count, context);
    mem_t<int> segments(num_segments, context);
    mem_t<float> output(num_segments, context);
    htod(input.data(), input_host, count);
    htod(segments.data(), segments_host, num_segments);
    segreduce(input.data(), count, segments.data(), num_segments,
      output.data(), plus_t<float>(), init, context);
    dtoh(output_host, output.data(), num_segments);
  } catch(cuda_exception_t& e) { return (int)e.result; }
  return finish();
}

} // extern "C"
