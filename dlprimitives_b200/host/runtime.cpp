// Context, ExecutionContext, TimingData, Tensor and the small name tables of definitions.hpp.
// This is host code above the C ABI: the only CUDA it touches is the runtime API for memory,
// streams and events.
#include <dlprim/context.hpp>
#include <dlprim/tensor.hpp>
#include "host_util.hpp"

#include <cuda_runtime.h>
#include <cstring>
#include <sstream>

namespace dlprim {

// ------------------------------------------------------------------------------------ definitions
DataType string_to_data_type(std::string const &s)
{
    if(s == "float" || s == "float32") return float_data;
    if(s == "float16" || s == "half") return half_data;
    if(s == "bfloat16") return bfloat16_data;
    if(s == "double" || s == "float64") return double_data;
    if(s == "int32" || s == "int") return int32_data;
    if(s == "uint32") return uint32_data;
    if(s == "int8") return int8_data;
    if(s == "uint8") return uint8_data;
    if(s == "int16") return int16_data;
    if(s == "uint16") return uint16_data;
    if(s == "int64") return int64_data;
    if(s == "uint64") return uint64_data;
    throw ValidationError("Unknown data type " + s);
}
std::string data_type_to_string(DataType dt)
{
    switch(dt) {
    case double_data: return "double";
    case int64_data: return "int64";
    case uint64_data: return "uint64";
    case float_data: return "float";
    case int32_data: return "int32";
    case uint32_data: return "uint32";
    case half_data: return "half";
    case bfloat16_data: return "bfloat16";
    case int16_data: return "int16";
    case uint16_data: return "uint16";
    case int8_data: return "int8";
    case uint8_data: return "uint8";
    }
    return "unknown";
}
StandardActivations activation_from_name(std::string const &name)
{
    if(name == "identity") return StandardActivations::identity;
    if(name == "relu") return StandardActivations::relu;
    if(name == "tanh") return StandardActivations::tanh;
    if(name == "sigmoid") return StandardActivations::sigmoid;
    if(name == "relu6") return StandardActivations::relu6;
    throw ValidationError("Invalid cativation name:" + name);
}
char const *activation_to_name(StandardActivations act)
{
    switch(act) {
    case StandardActivations::identity: return "identity";
    case StandardActivations::relu: return "relu";
    case StandardActivations::tanh: return "tanh";
    case StandardActivations::sigmoid: return "sigmoid";
    case StandardActivations::relu6: return "relu6";
    }
    throw ValidationError("Internal error invalid cativation");
}

namespace host {
void cuda_check(int err, char const *what)
{
    if(err != cudaSuccess) throw DeviceError(std::string(what) + ": " + cudaGetErrorString(cudaError_t(err)));
}
void status_check(int status)
{
    if(status == DLP_OK) return;
    std::string msg = dlp_last_error();
    switch(status) {
    case DLP_INVALID_ARGUMENT: throw ValidationError(msg);
    case DLP_NOT_IMPLEMENTED: throw NotImplementedError(msg);
    default: throw DeviceError(msg);
    }
}
} // namespace host
using host::cuda_check;

// ------------------------------------------------------------------------------------ Context
Context::Context(std::string const &dev_id)
{
    if(dev_id == "cpu")
        throw NotImplementedError("this library has no CPU context: the CUDA path has no CPU fallback");
    std::string s = dev_id;
    if(s.compare(0, 5, "cuda:") == 0) s = "0:" + s.substr(5);
    int p = 0, d = -1;
    std::istringstream ss(s);
    if(s.find(':') != std::string::npos) {
        char delim = 0;
        ss >> p >> delim >> d;
        if(!ss || delim != ':' || !ss.eof()) throw ValidationError("Invalid device identification expecting `platform_no:device_no` or `cuda:device_no`");
    }
    else {
        ss >> d;
        if(!ss || !ss.eof()) throw ValidationError("Invalid device identification expecting `platform_no:device_no` or `cuda:device_no`");
    }
    if(p != 0) throw ValidationError("No such platform " + std::to_string(p) + ": CUDA is platform 0");
    select(d);
}
Context::Context(ContextType dt, int platform, int device)
{
    if(dt == cpu) throw NotImplementedError("this library has no CPU context: the CUDA path has no CPU fallback");
    if(platform != 0) throw ValidationError("No such platform " + std::to_string(platform));
    select(device);
}
void Context::select(int device)
{
    int n = 0;
    cuda_check(cudaGetDeviceCount(&n), "cudaGetDeviceCount");
    if(device < 0 || device >= n) throw ValidationError("No such device " + std::to_string(device) + " of " + std::to_string(n));
    device_ = device;
    activate();
}
void Context::activate() const { cuda_check(cudaSetDevice(device_), "cudaSetDevice"); }
std::string Context::name() const
{
    cudaDeviceProp prop;
    cuda_check(cudaGetDeviceProperties(&prop, device_), "cudaGetDeviceProperties");
    return std::string(prop.name) + " on CUDA";
}
int Context::estimated_core_count() const
{
    int n = 0;
    cuda_check(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device_), "cudaDeviceGetAttribute");
    return n;
}

void ExecutionContext::finish() const { cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize"); }

// ------------------------------------------------------------------------------------ TimingData
TimingData::~TimingData() { reset(); }
void TimingData::enter(char const *name, cudaStream_t s)
{
    Section sec;
    sec.name = name;
    cuda_check(cudaEventCreate(&sec.start), "cudaEventCreate");
    cuda_check(cudaEventCreate(&sec.stop), "cudaEventCreate");
    sec.parent = stack_.empty() ? -1 : stack_.back();
    cuda_check(cudaEventRecord(sec.start, s), "cudaEventRecord");
    sections_.push_back(sec);
    stack_.push_back(int(sections_.size()) - 1);
}
void TimingData::leave(cudaStream_t s)
{
    if(stack_.empty()) throw ValidationError("TimingData::leave without enter");
    cuda_check(cudaEventRecord(sections_[stack_.back()].stop, s), "cudaEventRecord");
    stack_.pop_back();
}
void TimingData::resolve()
{
    for(Section &sec : sections_) {
        cuda_check(cudaEventSynchronize(sec.stop), "cudaEventSynchronize");
        float ms = 0;
        cuda_check(cudaEventElapsedTime(&ms, sec.start, sec.stop), "cudaEventElapsedTime");
        sec.time_ms = ms;
    }
}
void TimingData::reset()
{
    for(Section &sec : sections_) {
        if(sec.start) cudaEventDestroy(sec.start);
        if(sec.stop) cudaEventDestroy(sec.stop);
    }
    sections_.clear();
    stack_.clear();
}

// ------------------------------------------------------------------------------------ Tensor
struct Tensor::DeviceMem {
    void *ptr = nullptr;
    int device = 0;
    ~DeviceMem()
    {
        if(ptr) {
            int cur = 0;
            cudaGetDevice(&cur);
            if(cur != device) cudaSetDevice(device);
            cudaFree(ptr);
            if(cur != device) cudaSetDevice(cur);
        }
    }
};
struct Tensor::HostMem {
    void *ptr = nullptr;
    ~HostMem() { if(ptr) cudaFreeHost(ptr); }
};

Tensor::Tensor() : specs_(new TensorSpecs()) {}

Tensor::Tensor(Context &ctx, Shape const &s, DataType d, bool is_trainable) : specs_(new TensorSpecs(s, d, is_trainable))
{
    ctx.activate();
    size_t bytes = memory_size();
    capacity_ = bytes;
    mem_.reset(new DeviceMem());
    mem_->device = ctx.device_id();
    // at least one aligned block so that empty tensors still have a valid address
    cuda_check(cudaMalloc(&mem_->ptr, bytes < 256 ? 256 : bytes), "cudaMalloc");
    base_ = mem_->ptr;
}
Tensor::Tensor(void *device_ptr, size_t offset_elements, Shape const &s, DataType d, bool is_trainable)
    : specs_(new TensorSpecs(s, d, is_trainable)), base_(device_ptr), offset_(offset_elements)
{
    capacity_ = memory_size();
}
void Tensor::reshape(Shape const &ns)
{
    if(ns.total_size() * size_of_data_type(dtype()) > capacity_) throw ValidationError("respae: new size is larger than original");
    specs_.reset(new TensorSpecs(ns, dtype(), is_trainable()));
}
Tensor Tensor::sub_tensor(size_t offset, Shape const &s, DataType d, bool trainable) const
{
    size_t byte_offset = offset * size_of_data_type(d);
    size_t bytes = s.total_size() * size_of_data_type(d);
    if(byte_offset + bytes > capacity_) throw ValidationError("sub_tensor: the view does not fit the tensor");
    Tensor t;
    t.specs_.reset(new TensorSpecs(s, d, trainable));
    t.mem_ = mem_;
    size_t base_bytes = offset_ * size_of_data_type(dtype()) + byte_offset;
    DLPRIM_CHECK(base_bytes % size_of_data_type(d) == 0);
    t.base_ = base_;
    t.offset_ = base_bytes / size_of_data_type(d);
    t.capacity_ = bytes;       // the view's own block: the host mirror and reshape() stay inside it
    return t;
}
void *Tensor::host_data()
{
    if(!host_) {
        host_.reset(new HostMem());
        size_t bytes = capacity_ < 256 ? 256 : capacity_;
        cuda_check(cudaMallocHost(&host_->ptr, bytes), "cudaMallocHost");
        memset(host_->ptr, 0, bytes);
    }
    return host_->ptr;
}
void Tensor::to_device(ExecutionContext const &c, void *host_memory, bool sync)
{
    cuda_check(cudaMemcpyAsync(device_ptr(), host_memory, memory_size(), cudaMemcpyHostToDevice, c.stream()), "cudaMemcpyAsync H2D");
    if(sync) c.finish();
}
void Tensor::to_host(ExecutionContext const &c, void *host_memory, bool sync)
{
    cuda_check(cudaMemcpyAsync(host_memory, device_ptr(), memory_size(), cudaMemcpyDeviceToHost, c.stream()), "cudaMemcpyAsync D2H");
    if(sync) c.finish();
}
void Tensor::to_device(ExecutionContext const &c, bool sync) { to_device(c, host_data(), sync); }
void Tensor::to_host(ExecutionContext const &c, bool sync) { to_host(c, host_data(), sync); }

} // namespace dlprim
