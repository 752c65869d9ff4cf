"""B200-native fused sparse tree attention: GPU tree precompute + tree attention kernels.

Public surface (mirrors the reference's utils.py / fstattention.py):
  create_tree, create_full_attention_mask, create_fst_attention_kernel_inputs, DEPTH_MAPPING,
  MAX_ANCESTOR_MAPPING, fst_attention; plus build_tree_metadata / TreeMetadata for parent arrays
  and build_tree_topk, which grows the tree on the GPU from the heads' top-k scores
"""
from .utils import (DEPTH_MAPPING, MAX_ANCESTOR_MAPPING, TreeMetadata, build_tree_metadata,  # noqa: F401
                    create_fst_attention_kernel_inputs, create_full_attention_mask, create_tree,
                    build_tree_topk, dfs_order, dfs_order_device, lineage_from_parent, parent_from_lineage,
                    tree_topk_nodes)
from .fstattention import (clear_status, fst_attention, fst_attention_paged, last_status,  # noqa: F401
                           launch_plan)

__all__ = ["DEPTH_MAPPING", "MAX_ANCESTOR_MAPPING", "create_tree", "create_full_attention_mask",
           "TreeMetadata", "build_tree_metadata", "create_fst_attention_kernel_inputs",
           "lineage_from_parent", "parent_from_lineage", "dfs_order", "dfs_order_device", "fst_attention", "fst_attention_paged", "last_status", "clear_status", "launch_plan",
           "build_tree_topk", "tree_topk_nodes"]
