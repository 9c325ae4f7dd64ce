// Stand-ins, on platforms without Apple's Accelerate framework, for the handful of vDSP and
// vImage routines Honeycrisp's CPU backend calls (Sources/Honeycrisp/BackendCPU.swift:284-290,
// 337-339, 378-384, 464, 512, 666-680, 802, 1256, 2066; TensorElement.swift:262-277, 325-338) and
// for `autoreleasepool` (Backend.swift:151, DataUtil.swift:15, 61, 106).  Plain loops with the
// argument order of the originals; they make the package build on Linux, they are not fast.
// The matrix products that matter run in CUDABackend.
//
// Never compiled: there is no Swift toolchain where this repository is built.

#if !canImport(Accelerate)
  import Foundation

  public typealias vDSP_Length = UInt
  public typealias vDSP_Stride = Int

  @inline(__always)
  func autoreleasepool<T>(_ body: () throws -> T) rethrows -> T { try body() }

  // C = A + B
  func vDSP_vadd(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>, _ ib: vDSP_Stride,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ n: vDSP_Length
  ) { for i in 0..<Int(n) { c[i * ic] = a[i * ia] + b[i * ib] } }

  // C = A * B
  func vDSP_vmul(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>, _ ib: vDSP_Stride,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ n: vDSP_Length
  ) { for i in 0..<Int(n) { c[i * ic] = a[i * ia] * b[i * ib] } }

  // C = A / B; note that the divisor comes FIRST in vDSP's argument list.
  func vDSP_vdiv(
    _ b: UnsafePointer<Float>, _ ib: vDSP_Stride, _ a: UnsafePointer<Float>, _ ia: vDSP_Stride,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ n: vDSP_Length
  ) { for i in 0..<Int(n) { c[i * ic] = a[i * ia] / b[i * ib] } }

  // C = A - B; the subtrahend comes FIRST.
  func vDSP_vsub(
    _ b: UnsafePointer<Float>, _ ib: vDSP_Stride, _ a: UnsafePointer<Float>, _ ia: vDSP_Stride,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ n: vDSP_Length
  ) { for i in 0..<Int(n) { c[i * ic] = a[i * ia] - b[i * ib] } }

  // C = A + b
  func vDSP_vsadd(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ n: vDSP_Length
  ) { let s = b.pointee; for i in 0..<Int(n) { c[i * ic] = a[i * ia] + s } }

  // C = A * b
  func vDSP_vsmul(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ n: vDSP_Length
  ) { let s = b.pointee; for i in 0..<Int(n) { c[i * ic] = a[i * ia] * s } }

  // C = a / B
  func vDSP_svdiv(
    _ a: UnsafePointer<Float>, _ b: UnsafePointer<Float>, _ ib: vDSP_Stride,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ n: vDSP_Length
  ) { let s = a.pointee; for i in 0..<Int(n) { c[i * ic] = s / b[i * ib] } }

  // D = A * b + c
  func vDSP_vsmsa(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>,
    _ c: UnsafePointer<Float>, _ d: UnsafeMutablePointer<Float>, _ id: vDSP_Stride,
    _ n: vDSP_Length
  ) { let (m, s) = (b.pointee, c.pointee); for i in 0..<Int(n) { d[i * id] = a[i * ia] * m + s } }

  // D = A * B + C
  func vDSP_vma(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>, _ ib: vDSP_Stride,
    _ c: UnsafePointer<Float>, _ ic: vDSP_Stride, _ d: UnsafeMutablePointer<Float>,
    _ id: vDSP_Stride, _ n: vDSP_Length
  ) { for i in 0..<Int(n) { d[i * id] = a[i * ia] * b[i * ib] + c[i * ic] } }

  // D = (A + B) * C
  func vDSP_vam(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>, _ ib: vDSP_Stride,
    _ c: UnsafePointer<Float>, _ ic: vDSP_Stride, _ d: UnsafeMutablePointer<Float>,
    _ id: vDSP_Stride, _ n: vDSP_Length
  ) { for i in 0..<Int(n) { d[i * id] = (a[i * ia] + b[i * ib]) * c[i * ic] } }

  // c = sum of A
  func vDSP_sve(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ c: UnsafeMutablePointer<Float>,
    _ n: vDSP_Length
  ) {
    var acc: Float = 0
    for i in 0..<Int(n) { acc += a[i * ia] }
    c.pointee = acc
  }

  // C[m, n] = A[m, p] * B[p, n], all row-major with unit strides (the only use made of it).
  func vDSP_mmul(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ b: UnsafePointer<Float>, _ ib: vDSP_Stride,
    _ c: UnsafeMutablePointer<Float>, _ ic: vDSP_Stride, _ m: vDSP_Length, _ n: vDSP_Length,
    _ p: vDSP_Length
  ) {
    let (m, n, p) = (Int(m), Int(n), Int(p))
    for i in 0..<m {
      for j in 0..<n {
        var acc: Float = 0
        for k in 0..<p { acc += a[(i * p + k) * ia] * b[(k * n + j) * ib] }
        c[(i * n + j) * ic] = acc
      }
    }
  }

  // C[m, n] = transpose of A, where A is [n, m].
  func vDSP_mtrans(
    _ a: UnsafePointer<Float>, _ ia: vDSP_Stride, _ c: UnsafeMutablePointer<Float>,
    _ ic: vDSP_Stride, _ m: vDSP_Length, _ n: vDSP_Length
  ) {
    let (m, n) = (Int(m), Int(n))
    for i in 0..<m { for j in 0..<n { c[(i * n + j) * ic] = a[(j * m + i) * ia] } }
  }

  // vImage's planar float <-> half conversion, one row at a time; nearest-even on narrowing,
  // overflow to infinity (what the reference's tests expect, HCTestUtils/BackendTests.swift:81-83).
  struct vImage_Buffer {
    var data: UnsafeMutableRawPointer?
    var height: UInt
    var width: UInt
    var rowBytes: Int
  }
  let kvImageNoError = 0

  func vImageConvert_PlanarFtoPlanar16F(
    _ src: UnsafePointer<vImage_Buffer>, _ dst: UnsafePointer<vImage_Buffer>, _ flags: UInt32
  ) -> Int {
    guard let s = src.pointee.data, let d = dst.pointee.data else { return -1 }
    for row in 0..<Int(src.pointee.height) {
      let from = (s + row * src.pointee.rowBytes).assumingMemoryBound(to: Float.self)
      let to = (d + row * dst.pointee.rowBytes).assumingMemoryBound(to: Float16.self)
      for i in 0..<Int(src.pointee.width) { to[i] = Float16(from[i]) }
    }
    return kvImageNoError
  }

  func vImageConvert_Planar16FtoPlanarF(
    _ src: UnsafePointer<vImage_Buffer>, _ dst: UnsafePointer<vImage_Buffer>, _ flags: UInt32
  ) -> Int {
    guard let s = src.pointee.data, let d = dst.pointee.data else { return -1 }
    for row in 0..<Int(src.pointee.height) {
      let from = (s + row * src.pointee.rowBytes).assumingMemoryBound(to: Float16.self)
      let to = (d + row * dst.pointee.rowBytes).assumingMemoryBound(to: Float.self)
      for i in 0..<Int(src.pointee.width) { to[i] = Float(from[i]) }
    }
    return kvImageNoError
  }
#endif
