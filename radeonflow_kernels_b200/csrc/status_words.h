// Layout of the device status area shared by host and device code: four 32-bit words.
//   [0]    the first bounded device-side wait that expired: DeviceError code (1..6) in the low 8 bits, the
//          tag of the launch that recorded it above.  The other roles of that launch then give up their waits
//          after a few hundred polls, so a kernel that lost one role unwinds quickly; later launches (other
//          tags) are not affected.  The host entry points that read the word also clear it.
//   [1]    diagnostic flags that stop nothing (DeviceDiag), OR-ed in by kernels
//   [2,3]  wait limit in nanoseconds as one 64-bit value, written by the host (0 = the 2 s default)
#pragma once

namespace rf {

constexpr int kStatusWords = 4;
constexpr int kStatusDiagWord = 1;
constexpr int kStatusLimitWord = 2;
constexpr int kStatusTagShift = 8;          // status word 0 = code | (launch tag << 8); tags are 1 .. 2^22
constexpr int kStatusTagMask = (1 << 22) - 1;

}  // namespace rf
