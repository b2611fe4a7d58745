from .modeling_gpt_neo import (  # noqa: F401
    GPTNeoConfig, GPTNeoModel, GPTNeoForCausalLM, GPTNeoForSequenceClassification, GPTNeoLayerPolicy, GPTNeoSelfAttention, GPTNeoLocalSelfAttention, GPTNeoAttention, GPTNeoMLP, GPTNeoBlock, FusedGPTNeoSelfAttention, FusedGPTNeoLocalSelfAttention, FusedGPTNeoMLP, GPTNeoPreTrainedModel)
