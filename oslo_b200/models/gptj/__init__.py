from .modeling_gptj import (  # noqa: F401
    GPTJConfig, GPTJModel, GPTJForCausalLM, GPTJForSequenceClassification, GPTJLayerPolicy, GPTJAttention, GPTJMLP, GPTJBlock, FusedGPTJAttention, FusedGPTJMLP, GPTJPreTrainedModel)
