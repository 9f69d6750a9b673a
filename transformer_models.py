"""Model registry, configuration, portable layer and slicing helpers under the module name
the run scripts expect.  Everything is implemented in :mod:`terapipe_b200.models`."""
from terapipe_b200.models import *  # noqa: F401,F403
from terapipe_b200.models import (BATCH_CONFIGS, MODEL_CONFIGS, NEG_INF,  # noqa: F401
                                  ModelParallelMultiheadLMAttentionWithCache,
                                  ModelParallelTransformerLayer, MultiheadLMAttentionWithCache,
                                  SingleDeviceTransformer, TransformerConfig, TransformerLayer, assign_cache_,
                                  grid_slice_batch_and_sequence, load_grads, load_inputs,
                                  load_layers, merge_state_dicts, save_layers_and_inputs,
                                  slice_state_dict, uniform_slice_layers, uniform_slice_x)
