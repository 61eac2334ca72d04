// base:: enums, Status and error helpers with the names and numeric values of
// kuiper/include/base/base.h:11-176, without the glog dependency: the few logging / check
// macros the path needs are defined here on top of <cstdio>.  kDataTypeBf16 is new (the
// reference has Fp32, Int8, Int32, Fp16 only).
#ifndef KUIPER_INCLUDE_BASE_BASE_H_
#define KUIPER_INCLUDE_BASE_BASE_H_
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <ostream>
#include <string>

#define UNUSED(expr) \
  do {               \
    (void)(expr);    \
  } while (0)

// Precondition check in the spirit of glog's CHECK: reports and aborts.  Used only where
// the reference itself aborts (kernel free functions return void); everything that can
// fail at run time returns a base::Status instead.
#define KUIPER_CHECK(cond)                                                            \
  do {                                                                                \
    if (!(cond)) {                                                                    \
      std::fprintf(stderr, "Check failed: %s (%s:%d)\n", #cond, __FILE__, __LINE__); \
      std::abort();                                                                   \
    }                                                                                 \
  } while (0)

namespace model {
enum class ModelBufferType {
  kInputTokens = 0, kInputEmbeddings = 1, kOutputRMSNorm = 2, kKeyCache = 3, kValueCache = 4,
  kQuery = 5, kInputPos = 6, kScoreStorage = 7, kOutputMHA = 8, kAttnOutput = 9, kW1Output = 10,
  kW2Output = 11, kW3Output = 12, kFFNRMSNorm = 13, kForwardOutput = 15, kForwardOutputCPU = 16,
  kSinCache = 17, kCosCache = 18, kTempKey = 19, kTempValue = 20, kInputPosGPU = 21,
  kDecodeInput = 22, kInputPosPinned = 23, kArgmaxOutput = 24, kArgmaxOutputPinned = 25,
  kArgmaxPinned = 25, kKVCachePosGPU = 26, kKVCachePosPinned = 27,
  // paged KV-cache state (new): per-step device tensors the paged kernels read
  kBlockTable = 40, kSeqLens = 41, kSlotMapping = 42, kDecodeWorkspace = 43,
};
}  // namespace model

namespace base {
enum class DeviceType : uint8_t { kDeviceUnknown = 0, kDeviceCPU = 1, kDeviceCUDA = 2 };

enum class DataType : uint8_t {
  kDataTypeUnknown = 0,
  kDataTypeFp32 = 1,
  kDataTypeInt8 = 2,
  kDataTypeInt32 = 3,
  kDataTypeFp16 = 4,
  kDataTypeBf16 = 5,   // new
  kDataTypeInt64 = 6,  // new (slot mappings)
};

enum class ModelType : uint8_t { kModelTypeUnknown = 0, kModelTypeLLama2 = 1 };

inline size_t DataTypeSize(DataType t) {
  switch (t) {
    case DataType::kDataTypeFp32: return 4;
    case DataType::kDataTypeInt8: return 1;
    case DataType::kDataTypeInt32: return 4;
    case DataType::kDataTypeFp16: return 2;
    case DataType::kDataTypeBf16: return 2;
    case DataType::kDataTypeInt64: return 8;
    default: return 0;
  }
}

class NoCopyable {
 protected:
  NoCopyable() = default;
  ~NoCopyable() = default;
  NoCopyable(const NoCopyable&) = delete;
  NoCopyable& operator=(const NoCopyable&) = delete;
};

enum StatusCode : uint8_t {
  kSuccess = 0,
  kFunctionUnImplement = 1,
  kPathNotValid = 2,
  kModelParseError = 3,
  kInternalError = 5,
  kKeyValueHasExist = 6,
  kInvalidArgument = 7,
  // new: block pool exhausted (same value as KPX_ERR_OUT_OF_BLOCKS)
  kOutOfBlocks = 8,
};

enum class TokenizerType { kEncodeUnknown = -1, kEncodeSpe = 0, kEncodeBpe = 1 };

enum class AttentionType : uint8_t { kAttentionMHA = 0, kAttentionFlash1 = 1, kAttentionFlash2 = 2 };

inline const char* AttentionTypeName(AttentionType type) {
  switch (type) {
    case AttentionType::kAttentionMHA: return "MHA";
    case AttentionType::kAttentionFlash1: return "FlashAttention1";
    case AttentionType::kAttentionFlash2: return "FlashAttention2";
    default: return "Unknown";
  }
}

class Status {
 public:
  Status(int code = StatusCode::kSuccess, std::string err_message = "")
      : code_(code), message_(std::move(err_message)) {}
  Status(const Status&) = default;
  Status& operator=(const Status&) = default;
  Status& operator=(int code) {
    code_ = code;
    return *this;
  }
  bool operator==(int code) const { return code_ == code; }
  bool operator!=(int code) const { return code_ != code; }
  operator int() const { return code_; }
  operator bool() const { return code_ == kSuccess; }
  int32_t get_err_code() const { return code_; }
  const std::string& get_err_msg() const { return message_; }
  void set_err_msg(const std::string& err_msg) { message_ = err_msg; }

 private:
  int code_ = StatusCode::kSuccess;
  std::string message_;
};

namespace error {
#define STATUS_CHECK(call)                                                                       \
  do {                                                                                           \
    const base::Status& status = call;                                                           \
    if (!status) {                                                                               \
      std::fprintf(stderr, "Infer error\n File:%s Line:%d\n Error code:%d\n Error msg:%s\n",    \
                   __FILE__, __LINE__, int(status), status.get_err_msg().c_str());               \
      std::abort();                                                                              \
    }                                                                                            \
  } while (0)

inline Status Success(const std::string& m = "") { return Status{kSuccess, m}; }
inline Status FunctionNotImplement(const std::string& m = "") { return Status{kFunctionUnImplement, m}; }
inline Status PathNotValid(const std::string& m = "") { return Status{kPathNotValid, m}; }
inline Status ModelParseError(const std::string& m = "") { return Status{kModelParseError, m}; }
inline Status InternalError(const std::string& m = "") { return Status{kInternalError, m}; }
inline Status KeyHasExits(const std::string& m = "") { return Status{kKeyValueHasExist, m}; }
inline Status InvalidArgument(const std::string& m = "") { return Status{kInvalidArgument, m}; }
inline Status OutOfBlocks(const std::string& m = "") { return Status{kOutOfBlocks, m}; }
}  // namespace error

inline std::ostream& operator<<(std::ostream& os, const Status& x) {
  os << x.get_err_msg();
  return os;
}

}  // namespace base
#endif  // KUIPER_INCLUDE_BASE_BASE_H_
