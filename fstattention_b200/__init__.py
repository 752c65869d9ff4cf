"""B200-native fused sparse tree attention: GPU tree precompute + tree attention kernels.

Public surface (mirrors the reference's utils.py / fstattention.py):
  create_fst_attention_kernel_inputs, build_tree_metadata, TreeMetadata, fst_attention
"""
from .utils import (TreeMetadata, build_tree_metadata, create_fst_attention_kernel_inputs,  # noqa: F401
                    lineage_from_parent, parent_from_lineage)
from .fstattention import fst_attention, last_status  # noqa: F401

__all__ = ["TreeMetadata", "build_tree_metadata", "create_fst_attention_kernel_inputs",
           "lineage_from_parent", "parent_from_lineage", "fst_attention", "last_status"]
