// Stand-in for CRoaring (not installed here): the reference's utils.cuh only names the type.
#pragma once
namespace roaring {
class Roaring {};
}  // namespace roaring
