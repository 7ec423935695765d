// Stand-in for <gtest/gtest.h>, used only to compile the reference's test fixtures
// (tests/Arm/KaiLinearTest.hpp) as a library of their scalar reference functions.
// gtest is an empty submodule in the reference tree; only the base class is needed.
#pragma once
namespace testing {
class Test {
 public:
  virtual ~Test() = default;
  virtual void SetUp() {}
  virtual void TearDown() {}
};
}  // namespace testing
