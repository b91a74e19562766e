from .tensors import HeapTensorPool, nccl_dtype, tensor_from_ptr
