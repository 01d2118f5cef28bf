// Stands in for the reference's sideaware.cu when the reference's own C++ example (example_llmc_rope.cu, which
// does `#include "sideaware.cu"`, example_llmc_rope.cu:17) is built against THIS project's library instead: the
// recipe in oracle/Makefile copies this file next to the staged example under the name sideaware.cu.
// TEST INFRASTRUCTURE ONLY.  All it does is bring in the C ABI and the typed wrappers.
#include "sideaware.hpp"
