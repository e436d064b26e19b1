// Device selection and execution streams.
//
// The reference's Context picks an OpenCL platform:device or the CPU and its ExecutionContext wraps
// a command queue plus event lists (include/dlprim/context.hpp:128-299,309-431).  Here a Context is
// a CUDA device ordinal and an ExecutionContext is a cudaStream_t; ordering is the stream's order,
// which is what the reference's in-order queue gave its callers.  "P:D" strings keep parsing (the
// platform must be 0, D is the CUDA ordinal).  There is no CPU context in this library: "cpu" throws
// NotImplementedError -- the CPU path lives only in the separately built checker.
#pragma once
#include <dlprim/definitions.hpp>
#include <memory>
#include <string>
#include <vector>

typedef struct CUstream_st *cudaStream_t;
typedef struct CUevent_st *cudaEvent_t;

namespace dlprim {

/// Named timing sections measured with CUDA events on the stream (the reference's TimingData,
/// include/dlprim/context.hpp:23-94, measured OpenCL events and host wall-clock).
class DLPRIM_API TimingData {
public:
    struct Section {
        std::string name;
        cudaEvent_t start = nullptr, stop = nullptr;
        double time_ms = 0;
        int parent = -1;
    };
    ~TimingData();
    void enter(char const *name, cudaStream_t s);
    void leave(cudaStream_t s);
    /// Wait for the recorded events and fill Section::time_ms.
    void resolve();
    void reset();
    std::vector<Section> const &sections() const { return sections_; }
private:
    std::vector<Section> sections_;
    std::vector<int> stack_;
};

class DLPRIM_API Context {
public:
    enum ContextType { cpu = 0, ocl = 1, cuda = 1 };
    /// "D", "P:D" (P must be 0) or "cuda:D".
    Context(std::string const &dev_id);
    Context(ContextType dt = cuda, int platform = 0, int device = 0);
    bool is_cpu_context() const { return false; }
    bool is_opencl_context() const { return false; }
    bool is_cuda_context() const { return true; }
    ContextType context_type() const { return cuda; }
    int device_id() const { return device_; }
    std::string name() const;
    /// Number of streaming multiprocessors.
    int estimated_core_count() const;
    /// Make this device current for the calling thread.
    void activate() const;
private:
    void select(int device);
    int device_ = 0;
};

class DLPRIM_API ExecutionContext {
public:
    /// The default-constructed context runs on the legacy default stream.
    ExecutionContext() {}
    explicit ExecutionContext(cudaStream_t s) : stream_(s) {}
    cudaStream_t stream() const { return stream_; }
    void *stream_handle() const { return static_cast<void *>(stream_); }
    /// Block until everything enqueued on the stream is done.
    void finish() const;
    void enable_timing(std::shared_ptr<TimingData> p) { timing_ = p; }
    bool timing_enabled() const { return !!timing_; }
    std::shared_ptr<TimingData> timing() const { return timing_; }
    void enter(char const *name) const { if(timing_) timing_->enter(name, stream_); }
    void leave() const { if(timing_) timing_->leave(stream_); }
    /// The reference splits a context to wire events at the two ends of a multi-kernel operator
    /// (include/dlprim/context.hpp:192-197); on an in-order stream every step is this context itself.
    ExecutionContext generate_series_context(size_t, size_t) const { return *this; }
private:
    cudaStream_t stream_ = nullptr;
    std::shared_ptr<TimingData> timing_;
};

/// RAII timing scope, as the reference's ExecGuard (include/dlprim/context.hpp:435-449).
class ExecGuard {
public:
    ExecGuard(ExecutionContext const &e, char const *name) : e_(&e) { e.enter(name); }
    ~ExecGuard() { e_->leave(); }
    ExecGuard(ExecGuard const &) = delete;
    void operator=(ExecGuard const &) = delete;
private:
    ExecutionContext const *e_;
};

} // namespace dlprim
