"""B200-native batch similarity search behind VectorStoreKit's acceleration interface.

The compute lives in ``libvsk_cuda.so`` (hand-written sm_100a CUDA behind the C ABI declared in
``include/vsk_cuda.h``); this package is the host-side mirror of the reference's Swift types for
that path.  Importing the package does not need a GPU; opening a device does.
"""
from .engine import (CUDAAccelerationEngine, CUDAAcceleratorStrategy, CUDAComputeDevice, DeviceNotAvailable,
                     DeviceOutOfMemory, DimensionMismatch, DistanceMetric, EmptyInput, ExecutionFailed, FlatIndex,
                     InsufficientTrainingData, InvalidBufferSize, IVFIndex, KMeansClustering, QuantizedFlatIndex,
                     ScalarQuantizer, InvalidInput, NotTrained, SearchStrategy, Timeout,
                     UnsupportedOperation, VSKError, PATH_FP32_SCAN, PATH_TENSOR_RERANK, ImportFailed,
                     ExportFailed, import_index, load_index, ProductQuantizer, PQIndex, KMeansTrainer, sharded_slice)
from .store import InsertResult, IVFVectorIndex, SearchResult, VectorEntry, VectorStore
from .filters import (CompositeFilter, FilterBitmaskCompiler, FilterOperation, LogicalOperation, MetadataFilter,
                      VectorFilter)

__all__ = [n for n in dir() if not n.startswith("_")]
