// Tensor layout tags; same enumerators and order as portDNN's include/portdnn/data_format.h:31-43,
// filter_format.h:32-53, batch_format.h:32-44 and padding_mode.h:40.
#ifndef PORTDNN_B200_DATA_FORMAT_H_
#define PORTDNN_B200_DATA_FORMAT_H_
namespace sycldnn {
enum class DataFormat { NHWC, NCHW };
enum class FilterFormat { HWCF, FCHW, FHWC };
enum class BatchFormat { STRIDED, INTERLEAVED };
enum class PaddingMode { VALID, SAME };
}  // namespace sycldnn
#endif
