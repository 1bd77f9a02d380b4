"""Process-group plumbing: symmetric memory and handle exchange (bootstrap only;
no collective library call sits on a data path)."""
from .symm import (SymmetricHeap, pad_dim0_for_alignment, pad_to_granularity, vmm_granularity,
                   exchange_fds, resolve_handle_kind, tensor_from_ptr)

from .tensors import DistTensor, SingleOwnerTensor, create_dist_tensor, create_single_owner_tensor

__all__ = ["DistTensor", "SingleOwnerTensor", "create_dist_tensor", "create_single_owner_tensor",
           "SymmetricHeap", "pad_dim0_for_alignment", "pad_to_granularity", "vmm_granularity",
           "exchange_fds", "resolve_handle_kind", "tensor_from_ptr"]
