from .modeling_gptj import (  # noqa: F401
    GPTJConfig, GPTJModel, GPTJForCausalLM, GPTJForSequenceClassification, GPTJLayerPolicy, GPTJAttention, GPTJMLP, GPTJBlock, FusedGPTJAttention, FusedGPTJMLP, GPTJPreTrainedModel,
    fixed_pos_embedding, rotate_every_two, apply_rotary_pos_emb)
