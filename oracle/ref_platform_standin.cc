// Test infrastructure: a stand-in for the reference's Linux platform unit, which is the only
// user of <libunwind.h> (a header this image lacks). It provides the four functions declared
// in the reference's flint/lutil/platform.h and nothing else; the CPU GEMM that the oracle
// times and checks against never calls the stack walker.
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "lutil/platform.h"

namespace lut {

void *alloc32ByteAlignedMem(int64_t nbytes) {
  void *p = nullptr;
  size_t want = static_cast<size_t>(nbytes < 32 ? 32 : nbytes);
  if (posix_memalign(&p, 32, want) != 0) return nullptr;
  return p;
}

void free32ByteAlignedMem(void *p) { free(p); }

const char *getPathDelim() { return "/"; }

void printStackTrace() { fputs("(stack trace unavailable in the oracle build)\n", stderr); }

}  // namespace lut
