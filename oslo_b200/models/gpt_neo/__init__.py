from .modeling_gpt_neo import (  # noqa: F401
    GPTNeoConfig, GPTNeoModel, GPTNeoForCausalLM, GPTNeoForSequenceClassification, GPTNeoLayerPolicy, GPTNeoSelfAttention, GPTNeoLocalSelfAttention, GPTNeoAttention, GPTNeoMLP, GPTNeoBlock, FusedGPTNeoSelfAttention, FusedGPTNeoLocalSelfAttention, FusedGPTNeoMLP, GPTNeoPreTrainedModel)
from .convert_tf import load_tf_weights_in_gpt_neo  # noqa: F401
from .onnx_config import GPTNeoOnnxConfig  # noqa: F401
