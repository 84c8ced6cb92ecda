/*
 * CPU oracle for the load-balanced segmented-reduction path.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, what the
 * reference computes for segreduce / spmv / load-balancing search so that the
 * CUDA implementation can be checked against it. Nothing in the shipped
 * library calls it; only the tests, the smoke check and the CPU-baseline leg
 * of the benchmark do.
 *
 * Parity pins (see tests/test_oracle.py):
 *  - segreduce: the host loop of the reference's own test,
 *    tests/test_segreduce.cu:40-49, restated in oracle_segreduce_*; checked
 *    against closed-form sums of (index % 13) on the offsets that test
 *    generates, against golden vectors produced by running the reference's
 *    host-callable merge_path (tests/golden/), and on a GPU against the
 *    reference's CUDA build (oracle/_ref).
 *  - load-balancing search / partitions: src/moderngpu/cta_merge.hxx:8-29
 *    (merge_path) with bounds_upper as used by src/moderngpu/search.hxx:29-37,
 *    restated in oracle_merge_path_upper; checked against golden vectors
 *    produced by the reference's own function compiled for the host.
 *
 * Conventions shared by every function (reference: tests/test_segreduce.cu:
 * 16-22,41-42): `segments` holds num_segments START offsets, segments[0] == 0,
 * non-decreasing, values <= count; segment s is [segments[s], segments[s+1])
 * and the last segment ends at count.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORACLE_PLUS = 0, ORACLE_MAX = 1, ORACLE_MIN = 2 };

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static inline int64_t seg_end(const int32_t* segments, int num_segments,
  int64_t count, int s) {
  return (s + 1 < num_segments) ? (int64_t)segments[s + 1] : count;
}

/*
 * Host loop of tests/test_segreduce.cu:40-49:
 *   x = init; for rank in segment: x = rank ? op(x, y) : y;
 * i.e. `init` is the result of an empty segment only. `threads` > 1 spreads
 * segments over OpenMP threads (each segment is still folded serially).
 */
#define DEFINE_SEGREDUCE(NAME, T)                                              \
void NAME(const T* input, int64_t count, const int32_t* segments,             \
  int num_segments, T* output, T init, int op, int threads) {                 \
  (void)threads;                                                               \
  _Pragma("omp parallel for schedule(static, 4096) num_threads(threads) if(threads > 1)") \
  for(int s = 0; s < num_segments; ++s) {                                      \
    int64_t begin = segments[s];                                               \
    int64_t end = seg_end(segments, num_segments, count, s);                   \
    T x = init;                                                                \
    for(int64_t i = begin; i < end; ++i) {                                     \
      T y = input[i];                                                          \
      if(i == begin) x = y;                                                    \
      else if(ORACLE_PLUS == op) x = x + y;                                    \
      else if(ORACLE_MAX == op) x = (x < y) ? y : x;                           \
      else x = (y < x) ? y : x;                                                \
    }                                                                          \
    output[s] = x;                                                             \
  }                                                                            \
}

DEFINE_SEGREDUCE(oracle_segreduce_i32, int32_t)
DEFINE_SEGREDUCE(oracle_segreduce_i64, int64_t)
DEFINE_SEGREDUCE(oracle_segreduce_f32, float)
DEFINE_SEGREDUCE(oracle_segreduce_f64, double)

/*
 * Plus-reduction of fp32 (or fp64) items accumulated in a wider type, with
 * the sum of magnitudes per segment: the yardstick for floating-point
 * tolerance checks (|got - ref| <= tol * max(|ref|, sum |x|)).
 * Empty segments give init and a magnitude of 0.
 */
void oracle_segsum_f32_wide(const float* input, int64_t count,
  const int32_t* segments, int num_segments, double* sums, double* magnitudes,
  double init, int threads) {
  (void)threads;
  #pragma omp parallel for schedule(static, 4096) num_threads(threads) if(threads > 1)
  for(int s = 0; s < num_segments; ++s) {
    int64_t begin = segments[s];
    int64_t end = seg_end(segments, num_segments, count, s);
    double acc = 0, mag = 0;
    for(int64_t i = begin; i < end; ++i) {
      acc += (double)input[i];
      mag += input[i] < 0 ? -(double)input[i] : (double)input[i];
    }
    sums[s] = (end > begin) ? acc : init;
    magnitudes[s] = mag;
  }
}

void oracle_segsum_f64_wide(const double* input, int64_t count,
  const int32_t* segments, int num_segments, double* sums, double* magnitudes,
  double init, int threads) {
  (void)threads;
  #pragma omp parallel for schedule(static, 4096) num_threads(threads) if(threads > 1)
  for(int s = 0; s < num_segments; ++s) {
    int64_t begin = segments[s];
    int64_t end = seg_end(segments, num_segments, count, s);
    long double acc = 0, mag = 0;
    for(int64_t i = begin; i < end; ++i) {
      acc += (long double)input[i];
      mag += input[i] < 0 ? -(long double)input[i] : (long double)input[i];
    }
    sums[s] = (end > begin) ? (double)acc : init;
    magnitudes[s] = (double)mag;
  }
}

/*
 * Copies `input` into `placed` with the loop and schedule of the segreduce
 * above, so that every page of a freshly allocated `placed` is first touched
 * by the thread that will later reduce it (memory placement on hosts with
 * several NUMA nodes). Timing aid of the CPU baseline; computes nothing.
 */
void oracle_place_by_segments_f32(const float* input, int64_t count,
  const int32_t* segments, int num_segments, float* placed, int threads) {
  (void)threads;
  #pragma omp parallel for schedule(static, 4096) num_threads(threads) if(threads > 1)
  for(int s = 0; s < num_segments; ++s) {
    int64_t begin = s ? segments[s] : 0;
    int64_t end = seg_end(segments, num_segments, count, s);
    if(end > begin)
      memcpy(placed + begin, input + begin, (size_t)(end - begin) * sizeof(float));
  }
}

/*
 * transform_segreduce as the reference's test drives it
 * (tests/test_segreduce.cu:31-35,44-47): values are index % modulus.
 */
void oracle_segreduce_index_mod(int64_t count, const int32_t* segments,
  int num_segments, int32_t* output, int32_t init, int modulus) {
  for(int s = 0; s < num_segments; ++s) {
    int64_t begin = segments[s];
    int64_t end = seg_end(segments, num_segments, count, s);
    int32_t x = init;
    for(int64_t i = begin; i < end; ++i) {
      int32_t y = (int32_t)(i % modulus);
      x = (i == begin) ? y : x + y;
    }
    output[s] = x;
  }
}

/*
 * merge_path<bounds_upper> over (counting iterator, segments) with less-than:
 * src/moderngpu/cta_merge.hxx:8-29 called from src/moderngpu/search.hxx:33-36.
 * Returns how many items precede diagonal `diag` in the merge of
 * items 0..count-1 with the segment starts; a start sorts before the item of
 * equal index.
 */
int64_t oracle_merge_path_upper(int64_t count, const int32_t* segments,
  int64_t num_segments, int64_t diag) {
  int64_t begin = diag - num_segments;
  if(begin < 0) begin = 0;
  int64_t end = diag < count ? diag : count;
  while(begin < end) {
    int64_t mid = (begin + end) / 2;
    int64_t a_key = mid;
    int64_t b_key = segments[diag - 1 - mid];
    if(a_key < b_key) begin = mid + 1;
    else end = mid;
  }
  return begin;
}

/* load_balance_partitions: src/moderngpu/search.hxx:12-37. Writes
 * div_up(count + num_segments, spacing) + 1 values. */
int oracle_load_balance_partitions(int64_t count, const int32_t* segments,
  int num_segments, int spacing, int32_t* partitions) {
  int64_t total = count + num_segments;
  int n = (int)((total + spacing - 1) / spacing) + 1;
  for(int k = 0; k < n; ++k) {
    int64_t diag = (int64_t)spacing * k;
    if(diag > total) diag = total;
    partitions[k] = (int32_t)oracle_merge_path_upper(count, segments,
      num_segments, diag);
  }
  return n;
}

/*
 * Load-balancing search: for item i, seg = (number of starts <= i) - 1 and
 * rank = i - segments[seg] (src/moderngpu/cta_load_balance.hxx:128-170;
 * kernel_load_balance.hxx:78-86 stores seg). Either output may be NULL.
 */
void oracle_load_balance_search(int64_t count, const int32_t* segments,
  int num_segments, int32_t* seg_out, int32_t* rank_out) {
  int s = -1;
  for(int64_t i = 0; i < count; ++i) {
    while(s + 1 < num_segments && segments[s + 1] <= i) ++s;
    if(seg_out) seg_out[i] = s;
    if(rank_out) rank_out[i] = (int32_t)(i - (s >= 0 ? segments[s] : 0));
  }
}

/* interval_expand: output[i] = input[seg(i)], elements of elem_bytes bytes
 * (src/moderngpu/kernel_intervalmove.hxx:7-20). */
void oracle_interval_expand(const void* input, int elem_bytes, int64_t count,
  const int32_t* segments, int num_segments, void* output) {
  int s = -1;
  for(int64_t i = 0; i < count; ++i) {
    while(s + 1 < num_segments && segments[s + 1] <= i) ++s;
    if(s >= 0)
      memcpy((char*)output + i * elem_bytes,
        (const char*)input + (int64_t)s * elem_bytes, (size_t)elem_bytes);
  }
}

/*
 * CSR y = A * x (src/moderngpu/kernel_segreduce.hxx:285-298): products in the
 * matrix type, accumulated here in double; magnitudes as above.
 */
void oracle_spmv_f32(const float* matrix, const int32_t* columns,
  const float* x, int64_t nnz, const int32_t* row_starts, int rows,
  double* y, double* magnitudes) {
  for(int r = 0; r < rows; ++r) {
    int64_t begin = row_starts[r];
    int64_t end = seg_end(row_starts, rows, nnz, r);
    double acc = 0, mag = 0;
    for(int64_t i = begin; i < end; ++i) {
      double t = (double)matrix[i] * (double)x[columns[i]];
      acc += t;
      mag += t < 0 ? -t : t;
    }
    y[r] = acc;
    magnitudes[r] = mag;
  }
}

void oracle_spmv_f64(const double* matrix, const int32_t* columns,
  const double* x, int64_t nnz, const int32_t* row_starts, int rows,
  double* y, double* magnitudes) {
  for(int r = 0; r < rows; ++r) {
    int64_t begin = row_starts[r];
    int64_t end = seg_end(row_starts, rows, nnz, r);
    long double acc = 0, mag = 0;
    for(int64_t i = begin; i < end; ++i) {
      long double t = (long double)matrix[i] * (long double)x[columns[i]];
      acc += t;
      mag += t < 0 ? -t : t;
    }
    y[r] = (double)acc;
    magnitudes[r] = (double)mag;
  }
}

/* spmv in the matrix type itself, serial per row, rows over OpenMP threads:
 * the form the CPU baseline times. */
void oracle_spmv_f32_native(const float* matrix, const int32_t* columns,
  const float* x, int64_t nnz, const int32_t* row_starts, int rows, float* y,
  int threads) {
  (void)threads;
  #pragma omp parallel for schedule(static, 4096) num_threads(threads) if(threads > 1)
  for(int r = 0; r < rows; ++r) {
    int64_t begin = row_starts[r];
    int64_t end = seg_end(row_starts, rows, nnz, r);
    float acc = 0;
    for(int64_t i = begin; i < end; ++i) {
      float t = matrix[i] * x[columns[i]];
      acc = (i == begin) ? t : acc + t;
    }
    y[r] = acc;
  }
}

/*
 * lbs_segreduce with the functor f(index, seg, rank) = seg + rank that the
 * reference's test declares (tests/test_segreduce.cu:11-13) and a second
 * functor that exercises a per-segment cached value:
 * f(index, seg, rank, w) = values[index] * w[seg]   (fp32, wide accumulate).
 */
void oracle_lbs_segreduce_seg_plus_rank(int64_t count, const int32_t* segments,
  int num_segments, int32_t* output, int32_t init) {
  for(int s = 0; s < num_segments; ++s) {
    int64_t begin = segments[s];
    int64_t end = seg_end(segments, num_segments, count, s);
    int32_t x = init;
    for(int64_t i = begin; i < end; ++i) {
      int32_t y = (int32_t)(s + (i - begin));
      x = (i == begin) ? y : x + y;
    }
    output[s] = x;
  }
}

void oracle_lbs_segreduce_scaled_f32(const float* values, const float* weights,
  int64_t count, const int32_t* segments, int num_segments, double* sums,
  double* magnitudes, double init) {
  for(int s = 0; s < num_segments; ++s) {
    int64_t begin = segments[s];
    int64_t end = seg_end(segments, num_segments, count, s);
    double acc = 0, mag = 0;
    for(int64_t i = begin; i < end; ++i) {
      double t = (double)(values[i] * weights[s]);
      acc += t;
      mag += t < 0 ? -t : t;
    }
    sums[s] = (end > begin) ? acc : init;
    magnitudes[s] = mag;
  }
}
