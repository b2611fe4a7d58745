from .modeling_gpt2 import (  # noqa: F401
    GPT2Config, GPT2Model, GPT2LMHeadModel, GPT2DoubleHeadsModel, GPT2ForSequenceClassification, GPT2ForTokenClassification, GPT2LayerPolicy, GPT2Attention, GPT2MLP, GPT2Block, FusedGPT2Attention, FusedGPT2MLP, GPT2PreTrainedModel)
