// Null OpenCL C++ binding: test infrastructure only.
//
// The reference library's public headers include <CL/opencl.hpp>, but its
// CPU context never touches a device.  This header declares just enough of
// the cl:: surface for the reference host sources to compile unmodified; every
// call that would need a real OpenCL runtime throws cl::Error.  It is used
// only to build the CPU-context checker library under oracle/_ref.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>
#include <utility>

typedef int8_t cl_char;   typedef uint8_t cl_uchar;
typedef int16_t cl_short; typedef uint16_t cl_ushort;
typedef int32_t cl_int;   typedef uint32_t cl_uint;
typedef int64_t cl_long;  typedef uint64_t cl_ulong;
typedef float cl_float;   typedef double cl_double;
typedef cl_uint cl_bool;
typedef cl_ulong cl_command_queue_properties;
typedef cl_ulong cl_mem_flags;
typedef cl_ulong cl_device_type;
typedef void *cl_context; typedef void *cl_device_id; typedef void *cl_platform_id;
typedef void *cl_command_queue; typedef void *cl_mem; typedef void *cl_event;
typedef void *cl_kernel; typedef void *cl_program;

enum {
    CL_FALSE = 0, CL_TRUE = 1, CL_SUCCESS = 0,
    CL_MEM_READ_WRITE = 1,
    CL_DEVICE_TYPE_ALL = 0x7fffffff,
    CL_QUEUE_PROFILING_ENABLE = 2,
    CL_DEVICE_NAME = 0x1000, CL_DEVICE_VENDOR, CL_DEVICE_VENDOR_ID, CL_DEVICE_LOCAL_MEM_SIZE,
    CL_DEVICE_MAX_COMPUTE_UNITS, CL_DEVICE_EXTENSIONS, CL_DEVICE_PLATFORM, CL_DRIVER_VERSION,
    CL_DEVICE_MAX_WORK_GROUP_SIZE, CL_DEVICE_VERSION,
    CL_PLATFORM_NAME, CL_PLATFORM_VERSION, CL_PLATFORM_VENDOR,
    CL_QUEUE_CONTEXT, CL_QUEUE_DEVICE,
    CL_PROGRAM_BUILD_LOG, CL_PROGRAM_BINARIES, CL_PROGRAM_BINARY_SIZES,
    CL_PROFILING_COMMAND_START, CL_PROFILING_COMMAND_END, CL_PROFILING_COMMAND_QUEUED, CL_PROFILING_COMMAND_SUBMIT,
    CL_CONTEXT_DEVICES
};

namespace cl {
    class Error : public std::runtime_error {
    public:
        Error(cl_int e, char const *what = "OpenCL is not available in this build") : std::runtime_error(what), err_(e) {}
        cl_int err() const { return err_; }
    private:
        cl_int err_;
    };
    [[noreturn]] inline void unavailable() { throw Error(-1); }

    // Every query answers with a default-constructed value of whatever the caller asks for.
    struct AnyInfo {
        template<typename T> operator T() const { unavailable(); }
        template<typename T> bool operator==(T const &) const { unavailable(); }
        template<typename T> bool operator!=(T const &) const { unavailable(); }
        template<typename T> bool operator<(T const &) const { unavailable(); }
        template<typename T> bool operator>(T const &) const { unavailable(); }
        template<typename T> bool operator<=(T const &) const { unavailable(); }
        template<typename T> bool operator>=(T const &) const { unavailable(); }
    };

    template<typename Handle>
    class Wrapper {
    public:
        Wrapper() : h_(nullptr) {}
        explicit Wrapper(Handle h, bool = false) : h_(h) {}
        Handle operator()() const { return h_; }
        Handle get() const { return h_; }
        bool operator==(Wrapper const &o) const { return h_ == o.h_; }
        bool operator!=(Wrapper const &o) const { return h_ != o.h_; }
    protected:
        Handle h_;
    };

    // Result type of each getInfo<> query the reference makes.
    template<int N> struct InfoType { typedef cl_ulong type; };
    #define DLP_SHIM_STRING_INFO(name) template<> struct InfoType<name> { typedef std::string type; }
    DLP_SHIM_STRING_INFO(CL_DEVICE_NAME); DLP_SHIM_STRING_INFO(CL_DEVICE_VENDOR);
    DLP_SHIM_STRING_INFO(CL_DEVICE_EXTENSIONS); DLP_SHIM_STRING_INFO(CL_DRIVER_VERSION);
    DLP_SHIM_STRING_INFO(CL_DEVICE_VERSION); DLP_SHIM_STRING_INFO(CL_PLATFORM_NAME);
    DLP_SHIM_STRING_INFO(CL_PLATFORM_VERSION); DLP_SHIM_STRING_INFO(CL_PLATFORM_VENDOR);
    DLP_SHIM_STRING_INFO(CL_PROGRAM_BUILD_LOG);
    #undef DLP_SHIM_STRING_INFO
    template<> struct InfoType<CL_DEVICE_PLATFORM> { typedef cl_platform_id type; };
    template<> struct InfoType<CL_PROGRAM_BINARIES> { typedef std::vector<std::vector<unsigned char> > type; };

    class Device;
    class Platform : public Wrapper<cl_platform_id> {
    public:
        using Wrapper::Wrapper;
        static void get(std::vector<Platform> *p) { if(p) p->clear(); }
        void getDevices(cl_device_type, std::vector<Device> *d) const;
        template<int N> typename InfoType<N>::type getInfo() const { unavailable(); }
    };
    class Device : public Wrapper<cl_device_id> {
    public:
        using Wrapper::Wrapper;
        template<int N> typename InfoType<N>::type getInfo() const { unavailable(); }
    };
    inline void Platform::getDevices(cl_device_type, std::vector<Device> *d) const { if(d) d->clear(); }

    class Context : public Wrapper<cl_context> {
    public:
        using Wrapper::Wrapper;
        Context() {}
        Context(Device const &) { unavailable(); }
        Context(std::vector<Device> const &) { unavailable(); }
        template<int N> AnyInfo getInfo() const { return AnyInfo(); }
    };
    class Event : public Wrapper<cl_event> {
    public:
        using Wrapper::Wrapper;
        void wait() const { unavailable(); }
        template<int N> cl_ulong getProfilingInfo() const { unavailable(); }
    };
    class Buffer : public Wrapper<cl_mem> {
    public:
        using Wrapper::Wrapper;
        Buffer() {}
        Buffer(Context const &, cl_mem_flags, size_t, void * = nullptr) { unavailable(); }
    };
    struct LocalSpaceArg { size_t size_; };
    inline LocalSpaceArg Local(size_t s) { LocalSpaceArg a = { s }; return a; }

    class NDRange {
    public:
        NDRange() : n_(0) { s_[0] = s_[1] = s_[2] = 0; }
        NDRange(size_t a) : n_(1) { s_[0] = a; s_[1] = 1; s_[2] = 1; }
        NDRange(size_t a, size_t b) : n_(2) { s_[0] = a; s_[1] = b; s_[2] = 1; }
        NDRange(size_t a, size_t b, size_t c) : n_(3) { s_[0] = a; s_[1] = b; s_[2] = c; }
        size_t dimensions() const { return n_; }
        size_t operator[](int i) const { return s_[i]; }
        size_t const *get() const { return s_; }
        operator size_t const *() const { return s_; }
    private:
        size_t s_[3]; size_t n_;
    };
    static const NDRange NullRange;

    class Program : public Wrapper<cl_program> {
    public:
        using Wrapper::Wrapper;
        typedef std::vector<std::vector<unsigned char> > Binaries;
        typedef std::vector<std::string> Sources;
        Program() {}
        Program(Context const &, std::string const &, bool = false) { unavailable(); }
        Program(Context const &, Sources const &) { unavailable(); }
        Program(Context const &, std::vector<Device> const &, Binaries const &) { unavailable(); }
        void build(char const * = nullptr) const { unavailable(); }
        void build(std::vector<Device> const &, char const * = nullptr) const { unavailable(); }
        void build(Device const &, char const * = nullptr) const { unavailable(); }
        template<int N> typename InfoType<N>::type getInfo() const { unavailable(); }
        template<int N> typename InfoType<N>::type getBuildInfo(Device const &) const { unavailable(); }
    };
    typedef std::vector<std::pair<Device, std::string> > BuildLogType;
    class BuildError : public Error {
    public:
        BuildError() : Error(-2, "build") {}
        BuildLogType getBuildLog() const { return BuildLogType(); }
    };
    class Kernel : public Wrapper<cl_kernel> {
    public:
        using Wrapper::Wrapper;
        Kernel() {}
        Kernel(Program const &, char const *) { unavailable(); }
        Kernel(Program const &, std::string const &) { unavailable(); }
        template<typename T> void setArg(int, T const &) { unavailable(); }
        void setArg(int, size_t, void const *) { unavailable(); }
    };
    class CommandQueue : public Wrapper<cl_command_queue> {
    public:
        using Wrapper::Wrapper;
        CommandQueue() {}
        CommandQueue(Context const &, Device const &, cl_command_queue_properties = 0) { unavailable(); }
        template<int N> AnyInfo getInfo() const { return AnyInfo(); }
        void finish() const { unavailable(); }
        void flush() const { unavailable(); }
        void enqueueNDRangeKernel(Kernel const &, NDRange const &, NDRange const &, NDRange const & = NullRange,
                                  std::vector<Event> const * = nullptr, Event * = nullptr) const { unavailable(); }
        void enqueueReadBuffer(Buffer const &, cl_bool, size_t, size_t, void *,
                               std::vector<Event> const * = nullptr, Event * = nullptr) const { unavailable(); }
        void enqueueWriteBuffer(Buffer const &, cl_bool, size_t, size_t, void const *,
                                std::vector<Event> const * = nullptr, Event * = nullptr) const { unavailable(); }
        void enqueueCopyBuffer(Buffer const &, Buffer const &, size_t, size_t, size_t,
                               std::vector<Event> const * = nullptr, Event * = nullptr) const { unavailable(); }
        template<typename T>
        void enqueueFillBuffer(Buffer const &, T, size_t, size_t,
                               std::vector<Event> const * = nullptr, Event * = nullptr) const { unavailable(); }
        void enqueueBarrierWithWaitList(std::vector<Event> const * = nullptr, Event * = nullptr) const { unavailable(); }
        void enqueueMarkerWithWaitList(std::vector<Event> const * = nullptr, Event * = nullptr) const { unavailable(); }
    };
}
