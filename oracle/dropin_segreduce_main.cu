// Finite driver for the reference's tests/test_segreduce.cu built against this
// repository's headers. TEST INFRASTRUCTURE: the reference's source file is
// compiled unmodified (its own main(), which loops over 1000 seeds, is
// renamed on the command line) and its test_segreduce() is called here for a
// few seeds on the reference's own sizes (tests/test_segreduce.cu:67-73), so
// that the program ends by itself.
#include <moderngpu/kernel_segreduce.hxx>
#include <cstdlib>

void test_segreduce(int count, int num_segments, int seed,
  mgpu::context_t& context);

int main(int argc, char** argv) {
  int seeds = argc > 1 ? atoi(argv[1]) : 3;
  mgpu::standard_context_t context(false);
  const int count = 100000000, seg_size = 1000000;
  for(int seed = 0; seed < seeds; ++seed)
    test_segreduce(count, mgpu::div_up(count, seg_size), seed, context);
  printf("finished %d seeds\n", seeds);
  return 0;
}
