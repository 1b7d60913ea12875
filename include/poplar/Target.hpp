// Stand-in for poplar::Target: describes the GPU a graph is built for.  Only
// what the poplin path and its tools query is provided.
#ifndef poplar_Target_hpp
#define poplar_Target_hpp

#include <cstddef>
#include <string>

#include "poplar/Type.hpp"

namespace poplar {

class Target {
public:
  Target() = default;
  /// A CUDA device by ordinal; nothing is opened until a Graph is created.
  static Target createGPUTarget(int deviceOrdinal = 0) {
    Target t;
    t.device_ = deviceOrdinal;
    return t;
  }
  int getDeviceOrdinal() const { return device_; }
  /// The streaming multiprocessors play the part of the reference's tiles.
  unsigned getNumTiles() const { return 148; }
  unsigned getTilesPerIPU() const { return 148; }
  unsigned getNumIPUs() const { return 1; }
  std::size_t getTypeSize(const Type &t) const { return t.bytes(); }
  /// Peak arithmetic per SM and cycle, in the reference's terms: multiply-
  /// accumulates per cycle = conv units x vector width.  One SM's tensor core
  /// does 4096 dense fp16 (8192 fp8) MACs per cycle with fp32 accumulation;
  /// the CUDA cores 128 fp32 FMAs.
  unsigned getFloatVectorWidth() const { return 128; }
  unsigned getHalfVectorWidth() const { return 8; }
  unsigned getQuarterVectorWidth() const { return 16; }
  unsigned getFp16InFp16OutConvUnitsPerTile() const { return 512; }
  unsigned getFp16InFp32OutConvUnitsPerTile() const { return 512; }
  unsigned getFp32InFp32OutConvUnitsPerTile() const { return 0; }
  unsigned getFp8InFp16OutConvUnitsPerTile() const { return 512; }
  /// SM clock the cycle estimates refer to (the B200's maximum).
  double getTileClockFrequency() const { return 1.965e9; }
  std::string getTargetArchString() const { return "sm_100a"; }
  friend bool operator==(const Target &a, const Target &b) { return a.device_ == b.device_; }
  friend bool operator<(const Target &a, const Target &b) { return a.device_ < b.device_; }

private:
  int device_ = 0;
};

} // namespace poplar

#endif // poplar_Target_hpp
