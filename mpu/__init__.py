"""Model parallel utility interface under its historical package name.
Implemented in :mod:`terapipe_b200.parallel`."""
from terapipe_b200.parallel import *  # noqa: F401,F403
from terapipe_b200.parallel import (ColumnParallelLinear, ParallelEmbedding,  # noqa: F401
                                    RowParallelLinear, VocabParallelEmbedding, broadcast_data,
                                    checkpoint, copy_to_model_parallel_region,
                                    destroy_model_parallel, divide,
                                    gather_from_model_parallel_region, get_cuda_rng_tracker,
                                    get_data_parallel_group, get_data_parallel_rank,
                                    get_data_parallel_world_size, get_model_parallel_dst_rank,
                                    get_model_parallel_group, get_model_parallel_next_src_rank,
                                    get_model_parallel_prev_dst_rank, get_model_parallel_rank,
                                    get_model_parallel_src_rank, get_model_parallel_world_size,
                                    get_pipeline_parallel_group_rank,
                                    get_pipeline_parallel_pred_group,
                                    get_pipeline_parallel_succ_group,
                                    get_pipeline_parallel_world_size, initialize_model_parallel,
                                    model_parallel_cuda_manual_seed,
                                    model_parallel_is_initialized,
                                    reduce_from_model_parallel_region,
                                    scatter_to_model_parallel_region,
                                    split_tensor_along_last_dim, vocab_parallel_cross_entropy)
