// Stand-in for cereal's binary archive header.  The reference's graph container declares
// save/load members that name the two archive classes (include/coalsack/core/subgraph.h:145-154);
// nothing here ever serializes a graph, so the classes accept anything and do nothing.
// Test infrastructure only.
#pragma once
#include <iosfwd>
namespace cereal {
class BinaryOutputArchive {
 public:
  explicit BinaryOutputArchive(std::ostream&) {}
  template <typename... T>
  BinaryOutputArchive& operator()(T&&...) { return *this; }
};
class BinaryInputArchive {
 public:
  explicit BinaryInputArchive(std::istream&) {}
  template <typename... T>
  BinaryInputArchive& operator()(T&&...) { return *this; }
};
}  // namespace cereal
