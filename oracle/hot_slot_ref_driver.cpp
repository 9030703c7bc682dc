// Driver that runs the REFERENCE's own hot-slot bitmap selector on the host.
//
// TEST INFRASTRUCTURE ONLY. The selector source is not copied: the Makefile adds the
// reference checkout's csrc/operators/lidu/op_kernel directory to the include path and this
// file includes hot_slot_selection.h from there, with the five stub macros the reference's
// own CPU test uses (tests/operators/lidu/test_hot_slot_selection.py:17-42).
// stdin: lines "budget begin n word0 word1 ..."; stdout: the n selected slots per line.
#include <cstdint>
#include <iostream>
#include <vector>
#define __simt_callee__
#define __simt_vf__
#define __aicore__
#define __ubuf__
#define LAUNCH_BOUND(x)
namespace AscendC { namespace Simt {
unsigned tid;
unsigned GetThreadIdx() { return tid; }
unsigned GetThreadNum() { return 512; }
}}
#include "hot_slot_selection.h"

int main() {
  unsigned budget, begin, n;
  while (std::cin >> budget >> begin >> n) {
    std::vector<uint32_t> bits((budget + 31) / 32);
    for (auto& v : bits) std::cin >> v;
    const unsigned first = (budget - 1) / 32 - begin / 32 + 1, second = begin ? (begin - 1) / 32 + 1 : 0;
    std::vector<int32_t> count(first + second), prefix(first + second), out(n, -1);
    for (unsigned t = 0; t < 512; ++t) {
      AscendC::Simt::tid = t;
      kvip_hot_slots::CountAvailableBitmapWordsBody(bits.data(), count.data(), budget, begin, first, second);
    }
    unsigned total = 0;
    for (unsigned i = 0; i < count.size(); ++i) { prefix[i] = static_cast<int32_t>(total); total += count[i]; }
    for (unsigned t = 0; t < 512; ++t) {
      AscendC::Simt::tid = t;
      kvip_hot_slots::WriteAvailableBitmapSlotsBody(bits.data(), count.data(), prefix.data(), out.data(), budget,
                                                    begin, first, second, n, 0);
    }
    for (auto v : out) std::cout << v << ' ';
    std::cout << '\n';
  }
}
