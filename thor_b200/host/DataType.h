// DataType tokens of the host layer; integer values equal ThorImplementation::DataType
// (DeepLearning/Implementation/Tensor/DataType.h:7-26) and the thor_b200_dtype enum of the C ABI.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace ThorB200 {

enum class DataType : int {
    FP16 = 10, FP32 = 11, FP64 = 12, INT8 = 13, INT16 = 14, INT32 = 15, INT64 = 16, UINT8 = 17, UINT16 = 18, UINT32 = 19,
    UINT64 = 20, BOOLEAN = 21, FP8_E4M3 = 22, FP8_E5M2 = 23, BF16 = 24,
};

inline size_t dataTypeSize(DataType dt) {
    switch (dt) {
        case DataType::FP16: case DataType::BF16: case DataType::INT16: case DataType::UINT16: return 2;
        case DataType::FP32: case DataType::INT32: case DataType::UINT32: return 4;
        case DataType::FP64: case DataType::INT64: case DataType::UINT64: return 8;
        default: return 1;
    }
}

inline const char* dataTypeName(DataType dt) {
    switch (dt) {
        case DataType::FP16: return "fp16"; case DataType::FP32: return "fp32"; case DataType::FP64: return "fp64";
        case DataType::INT8: return "int8"; case DataType::INT16: return "int16"; case DataType::INT32: return "int32";
        case DataType::INT64: return "int64"; case DataType::UINT8: return "uint8"; case DataType::UINT16: return "uint16";
        case DataType::UINT32: return "uint32"; case DataType::UINT64: return "uint64"; case DataType::BOOLEAN: return "boolean";
        case DataType::FP8_E4M3: return "fp8_e4m3"; case DataType::FP8_E5M2: return "fp8_e5m2"; case DataType::BF16: return "bf16";
    }
    return "unknown";
}

// Floating types a fused stage can compute on (isSupportedFusionFloatingType in
// Utilities/Expression/ExpressionDTypeResolution.cpp).
inline bool isFusionFloat(DataType dt) {
    return dt == DataType::FP16 || dt == DataType::BF16 || dt == DataType::FP32 || dt == DataType::FP8_E4M3 || dt == DataType::FP8_E5M2;
}
inline bool isFp8(DataType dt) { return dt == DataType::FP8_E4M3 || dt == DataType::FP8_E5M2; }

}  // namespace ThorB200
