// Basic vocabulary of the host API: error types, data types, activations, convolution settings.
// Same names and meaning as the reference's include/dlprim/definitions.hpp (errors :38-75,
// DataType :77-90, StandardActivations :278-284, Convolution2DConfigBase :313-321), so code written
// against the reference compiles against this library; only fp32 compute exists on this path.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>

#define DLPRIM_API __attribute__((visibility("default")))

namespace dlprim {
namespace json { class value; }

class DLPRIM_API Error : public std::runtime_error {
public:
    explicit Error(std::string const &v) : std::runtime_error(v) {}
};
class DLPRIM_API NotImplementedError : public Error {
public:
    explicit NotImplementedError(std::string const &v) : Error(v) {}
};
class DLPRIM_API ValidationError : public Error {
public:
    explicit ValidationError(std::string const &v) : Error(v) {}
};
/// A CUDA runtime or kernel failure (the reference surfaces cl::Error here).
class DLPRIM_API DeviceError : public Error {
public:
    explicit DeviceError(std::string const &v) : Error(v) {}
};

#define DLPRIM_CHECK(x) \
    do { if(!(x)) throw ::dlprim::ValidationError(std::string("Failed " #x " at " __FILE__ ":") + std::to_string(__LINE__)); } while(0)

// type code = log2(size)+1 in the low 3 bits, kind in the next bits (same numbering as the reference)
enum DataType {
    double_data = 4 + (0 << 3), int64_data = 4 + (2 << 3), uint64_data = 4 + (3 << 3),
    float_data = 3 + (0 << 3), int32_data = 3 + (2 << 3), uint32_data = 3 + (3 << 3),
    half_data = 2 + (0 << 3), bfloat16_data = 2 + (1 << 3), int16_data = 2 + (2 << 3), uint16_data = 2 + (3 << 3),
    int8_data = 1 + (2 << 3), uint8_data = 1 + (3 << 3),
};
inline bool is_floating_point_data_type(DataType d) { return (d >> 3) < 2; }
constexpr int size_of_data_type(DataType d) { return 1 << ((d & 0x7) - 1); }
DLPRIM_API DataType string_to_data_type(std::string const &s);
DLPRIM_API std::string data_type_to_string(DataType dt);

template<typename T> struct TypeTraits;
template<> struct TypeTraits<float> { static constexpr DataType data_type = float_data; };
template<> struct TypeTraits<double> { static constexpr DataType data_type = double_data; };
template<> struct TypeTraits<int32_t> { static constexpr DataType data_type = int32_data; };
template<> struct TypeTraits<int64_t> { static constexpr DataType data_type = int64_data; };
template<> struct TypeTraits<uint8_t> { static constexpr DataType data_type = uint8_data; };

static constexpr int max_tensor_dim = 8;

enum class StandardActivations : int { identity = 0, relu = 1, tanh = 2, sigmoid = 3, relu6 = 4 };
DLPRIM_API StandardActivations activation_from_name(std::string const &name);
DLPRIM_API char const *activation_to_name(StandardActivations act);

enum class CalculationsMode { train, predict };
enum class GemmOpMode { forward = 1, backward_filter = 2, backward_data = 3 };

struct Convolution2DConfigBase {
    int channels_in = -1;
    int channels_out = -1;
    int kernel[2] = {1, 1};
    int stride[2] = {1, 1};
    int dilate[2] = {1, 1};
    int pad[2] = {0, 0};
    int groups = 1;
};

} // namespace dlprim
