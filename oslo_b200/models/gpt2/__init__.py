from .modeling_gpt2 import (  # noqa: F401
    GPT2Config, GPT2Model, GPT2LMHeadModel, GPT2DoubleHeadsModel, GPT2ForSequenceClassification, GPT2ForTokenClassification, GPT2LayerPolicy, GPT2Attention, GPT2MLP, GPT2Block, FusedGPT2Attention, FusedGPT2MLP, GPT2PreTrainedModel)
from .convert_tf import load_tf_weights_in_gpt2, tf_name_to_key  # noqa: F401
from .onnx_config import GPT2OnnxConfig  # noqa: F401
