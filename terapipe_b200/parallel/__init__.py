"""Tensor / pipeline / data parallel utility interface (the reference's ``mpu``)."""
from .cross_entropy import vocab_parallel_cross_entropy
from .data import broadcast_data
from .initialize import (destroy_model_parallel, get_data_parallel_group,
                         get_data_parallel_rank, get_data_parallel_world_size,
                         get_model_parallel_dst_rank, get_model_parallel_group,
                         get_model_parallel_next_src_rank, get_model_parallel_prev_dst_rank,
                         get_model_parallel_rank, get_model_parallel_src_rank,
                         get_model_parallel_world_size, get_pipeline_next_rank,
                         get_pipeline_parallel_group, get_pipeline_parallel_group_rank,
                         get_pipeline_parallel_pred_group, get_pipeline_parallel_succ_group,
                         get_pipeline_parallel_world_size, get_pipeline_prev_rank,
                         get_topology, initialize_model_parallel,
                         model_parallel_is_initialized)
from .layers import (ColumnParallelLinear, ParallelEmbedding, RowParallelLinear,
                     VocabParallelEmbedding)
from .mappings import (copy_to_model_parallel_region, gather_from_model_parallel_region,
                       gather_from_sequence_parallel_region, reduce_from_model_parallel_region,
                       reduce_scatter_to_sequence_parallel_region, scatter_to_model_parallel_region,
                       scatter_to_sequence_parallel_region)
from .random import checkpoint, get_cuda_rng_tracker, model_parallel_cuda_manual_seed
from .topology import Topology
from .utils import VocabUtility, divide, ensure_divisibility, split_tensor_along_last_dim
