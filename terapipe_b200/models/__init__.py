from .config import BATCH_CONFIGS, MODEL_CONFIGS, NEG_INF, TransformerConfig
from .layers import (ModelParallelMultiheadLMAttentionWithCache, ModelParallelTransformerLayer,
                     MultiheadLMAttentionWithCache, SingleDeviceTransformer, TransformerLayer,
                     assign_cache_)
from .slicing import (grid_slice_batch_and_sequence, load_grads, load_inputs, load_layers,
                      merge_state_dicts, save_layers_and_inputs, slice_state_dict,
                      uniform_slice_layers, uniform_slice_x)
