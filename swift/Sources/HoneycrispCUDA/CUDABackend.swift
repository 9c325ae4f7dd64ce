// CUDABackend: a Honeycrisp `Backend` whose matrix products run in libhccuda on a B200.
//
// Written against the reference's interfaces as read from its sources; it has NOT been
// compiled (no Swift toolchain exists where this repository is built).
//
// It is a `BackendWrapper` (Sources/Honeycrisp/BackendWrapper.swift:9) around the CPU backend:
// the two hot-path primitives, `matmul` (Backend.swift:650-658) and `batchedMatmul` (:661-669),
// are overridden and run on the GPU, and so are `cast` between the float types and `constant`;
// every other primitive - collection, random sampling, elementwise and reduction ops - falls
// through to the wrapped backend, so that
// `Backend.defaultBackend = try CUDABackend()` is a drop-in: tensors can be created, a Linear
// layer runs forward and backward, and the reference's own tests pass through it.  Operands that
// arrive as another backend's `Tensor.Data` are staged to the device through `onCPU`, as
// MPSBackend does (BackendMPS.swift:585-620); results are `CUDAData`, which the wrapped backend
// reads through `onCPU` when a CPU op consumes them.  Consecutive products stay on the device.
//
// CHCCuda is the module map over include/hc_cuda.h (Sources/CHCCuda/module.modulemap; put the
// header's directory on the include path and libhccuda.so on the linker path).

import CHCCuda
import Foundation
import HCBacktrace
import Honeycrisp

/// Device buffer: the `Tensor.Data` conformer of this backend (Tensor.swift:69-85).
public final class CUDAData: Tensor.Data, @unchecked Sendable {
  public let backend: CUDABackend
  public let pointer: UnsafeMutableRawPointer
  public let byteCount: Int

  private let lock = NSLock()
  /// Completion marker recorded after the work that fills this buffer.
  private var event: OpaquePointer?
  /// Operands of that work; kept until the work is known to have run.
  private var inputs: [any Tensor.Data] = []

  init(backend: CUDABackend, byteCount: Int) throws {
    self.backend = backend
    self.byteCount = byteCount
    var ptr: UnsafeMutableRawPointer? = nil
    // bytes == 0 allocates one byte, as MPSBackend does (BackendMPS.swift:538-540).
    let st = hc_alloc(backend.ctx, byteCount, &ptr)
    guard st == HC_OK, let p = ptr else { throw BackendError.allocationFailed(byteCount) }
    self.pointer = p
  }

  deinit {
    if let ev = event { hc_event_destroy(ev) }
    // Stream-ordered free: runs after everything already enqueued that uses the buffer.
    _ = hc_free(backend.ctx, pointer)
  }

  /// Called once, by the operation that produces the buffer, before the buffer is published.
  func produced(by inputs: [any Tensor.Data]) throws {
    var ev: OpaquePointer? = nil
    try backend.check(hc_event_record(backend.ctx, &ev))
    lock.lock()
    if let old = event { hc_event_destroy(old) }
    event = ev
    self.inputs = inputs
    lock.unlock()
  }

  private func currentEvent() -> OpaquePointer? {
    lock.lock()
    defer { lock.unlock() }
    return event
  }

  public func wait() async throws {
    let ev = currentEvent()
    let backend = self.backend
    try await backend.offload {
      if let ev = ev { try backend.check(hc_event_wait(ev)) } else { try backend.check(hc_sync(backend.ctx)) }
    }
    lock.lock()
    inputs = []
    lock.unlock()
  }

  public func onCPU<T>(_ fn: (_: UnsafeRawPointer) async throws -> T) async throws -> T {
    let host = UnsafeMutableRawPointer.allocate(byteCount: max(1, byteCount), alignment: 16)
    defer { host.deallocate() }
    let (ctx, src, n) = (backend.ctx, pointer, byteCount)
    let backend = self.backend
    // Read back on the side stream and wait for that copy only: products enqueued after this
    // tensor keep running (hc_sync would wait for all of them).
    try await backend.offload {
      var done: OpaquePointer? = nil
      try backend.check(hc_d2h_async(ctx, host, src, n, &done))
      defer { hc_event_destroy(done) }
      try backend.check(hc_event_wait(done))
    }
    return try await fn(UnsafeRawPointer(host))
  }

  public func mutateOnCPU<T>(_ fn: (_: UnsafeMutableRawPointer) async throws -> T) async throws -> T {
    let host = UnsafeMutableRawPointer.allocate(byteCount: max(1, byteCount), alignment: 16)
    defer { host.deallocate() }
    let (ctx, dev, n) = (backend.ctx, pointer, byteCount)
    let backend = self.backend
    try await backend.offload {
      var done: OpaquePointer? = nil
      try backend.check(hc_d2h_async(ctx, host, dev, n, &done))
      defer { hc_event_destroy(done) }
      try backend.check(hc_event_wait(done))
    }
    let result = try await fn(host)
    try await backend.offload {
      // Ordered after everything enqueued so far (earlier readers of the buffer are done); later
      // work on the context is told to wait for the upload, the host only waits for the copy to
      // leave `host`, which is freed on return.
      var done: OpaquePointer? = nil
      try backend.check(hc_h2d_async(ctx, dev, host, n, &done))
      defer { hc_event_destroy(done) }
      try backend.check(hc_enqueue_wait(ctx, done))
      try backend.check(hc_event_wait(done))
    }
    return result
  }
}

open class CUDABackend: BackendWrapper, @unchecked Sendable {
  let ctx: OpaquePointer
  /// Calls that may block (syncs, copies) leave the cooperative pool, as the reference backends
  /// do with their WorkerThread (Backend.swift:135-163, BackendCPU.swift:235-248).
  private let worker = Backend.WorkerThread()

  /// `wrapping` serves every primitive this class does not override.
  public init(device: Int = 0, wrapping: Backend = CPUBackend.global) throws {
    var c: OpaquePointer? = nil
    let st = hc_init(Int32(device), &c)
    guard st == HC_OK, let ctx = c else {
      throw BackendError.kernelFailed("hc_init(device: \(device)): \(String(cString: hc_status_string(st)))")
    }
    self.ctx = ctx
    super.init(wrapping: wrapping)
  }

  deinit { hc_destroy(ctx) }

  /// Run a blocking piece of work (a sync, a copy) on the backend's worker thread and resume
  /// the caller with its result - the same hand-off CPUBackend.serialize makes
  /// (BackendCPU.swift:235-248) over Backend.WorkerThread.schedule (Backend.swift:160-162).
  func offload<T>(_ fn: @escaping @Sendable () throws -> T) async throws -> T {
    try await withCheckedThrowingContinuation { continuation in
      worker.schedule {
        do {
          continuation.resume(returning: try fn())
        } catch {
          continuation.resume(throwing: error)
        }
      }
    }
  }

  func check(_ st: hc_status) throws {
    if st == HC_OK { return }
    // hc_copy_last_error takes the context's lock; hc_last_error would read the message while
    // another thread's call may be writing it.
    var buf = [CChar](repeating: 0, count: 256)
    hc_copy_last_error(ctx, &buf, buf.count)
    let msg = String(cString: buf)
    switch st {
    case HC_ERR_ALLOCATION_FAILED: throw BackendError.allocationFailed(0)
    case HC_ERR_NOT_IMPLEMENTED: throw BackendError.notImplemented(msg)
    default: throw BackendError.kernelFailed(msg.isEmpty ? String(cString: hc_status_string(st)) : msg)
    }
  }

  /// Operands of another backend's Data type are staged through onCPU, as
  /// MPSBackend.gpuBuffer does (BackendMPS.swift:585-620).
  func deviceOperand(_ x: Tensor.Data, byteCount n: Int) async throws -> CUDAData {
    if let d = x as? CUDAData, d.backend === self { return d }
    let out = try CUDAData(backend: self, byteCount: n)
    try await x.onCPU { host in
      try await self.offload {
        try self.check(hc_h2d(self.ctx, out.pointer, host, n))
        try self.check(hc_sync(self.ctx))   // `host` is only valid inside this closure
      }
    }
    return out
  }

  func hcDType(_ dtype: Tensor.DType) -> hc_dtype? {
    switch dtype {
    case .float16: return HC_F16
    case .float32: return HC_F32
    default: return nil
    }
  }

  override open func matmul(
    a: Tensor.Data, transA: Bool, b: Tensor.Data, transB: Bool, transOut: Bool, rows: Int,
    inner: Int, cols: Int, dtype: Tensor.DType
  ) async throws -> Tensor.Data {
    try await batchedMatmul(
      matrixCount: 1, a: a, transA: transA, b: b, transB: transB, transOut: transOut, rows: rows,
      inner: inner, cols: cols, dtype: dtype)
  }

  override open func batchedMatmul(
    matrixCount: Int, a: Tensor.Data, transA: Bool, b: Tensor.Data, transB: Bool, transOut: Bool,
    rows: Int, inner: Int, cols: Int, dtype: Tensor.DType
  ) async throws -> Tensor.Data {
    guard let dt = hcDType(dtype) else {
      // int64 products are legal in the reference and served by its CPU loop (BackendCPU.swift:1307-1311).
      return try await wrapped.batchedMatmul(
        matrixCount: matrixCount, a: a, transA: transA, b: b, transB: transB, transOut: transOut,
        rows: rows, inner: inner, cols: cols, dtype: dtype)
    }
    let aCount = matrixCount * rows * inner * dtype.byteSize
    let bCount = matrixCount * inner * cols * dtype.byteSize
    // Same size checks MPSBackend makes before encoding (BackendMPS.swift:2221-2230).
    alwaysAssert(a.byteCount >= aCount, "matmul: operand a is too small")
    alwaysAssert(b.byteCount >= bCount, "matmul: operand b is too small")
    let aBuf = try await deviceOperand(a, byteCount: aCount)
    let bBuf = try await deviceOperand(b, byteCount: bCount)
    let out = try CUDAData(backend: self, byteCount: matrixCount * rows * cols * dtype.byteSize)
    // Enqueue only; the product runs asynchronously and `out.wait()` is the sync point.
    try check(
      hc_batched_matmul(
        ctx, dt, Int64(matrixCount), aBuf.pointer, transA ? 1 : 0, bBuf.pointer, transB ? 1 : 0,
        transOut ? 1 : 0, Int64(rows), Int64(inner), Int64(cols), out.pointer))
    try out.produced(by: [aBuf, bBuf])
    return out
  }

  /// `Backend.constant` (Backend.swift:787-791) for the float types is a fill on the device, so that
  /// `Tensor(zeros:)`/`Tensor(ones:)` operands of a product never cross the host link.
  override open func constant<T: TensorElement>(_ value: T, count: Int, dtype: Tensor.DType)
    async throws -> Tensor.Data
  {
    guard let dt = hcDType(dtype) else {
      return try await wrapped.constant(value, count: count, dtype: dtype)
    }
    let out = try CUDAData(backend: self, byteCount: count * dtype.byteSize)
    try check(hc_constant(ctx, dt, value.toFloat(), Int64(count), out.pointer))
    try out.produced(by: [])
    return out
  }

  /// `Backend.cast` between the two float types stays on the device when its input lives there
  /// (Linear's `weight.cast(castParams)`, Trainable.swift:540); anything else goes to the wrapped backend.
  override open func cast(_ a: Tensor.Data, count: Int, inType: Tensor.DType, outType: Tensor.DType)
    async throws -> Tensor.Data
  {
    guard let d = a as? CUDAData, d.backend === self, let from = hcDType(inType), let to = hcDType(outType)
    else {
      return try await wrapped.cast(a, count: count, inType: inType, outType: outType)
    }
    let out = try CUDAData(backend: self, byteCount: count * outType.byteSize)
    try check(hc_cast(ctx, from, to, d.pointer, Int64(count), out.pointer))
    try out.produced(by: [d])
    return out
  }
}
