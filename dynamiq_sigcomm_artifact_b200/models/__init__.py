"""Model families: GPT-2 (causal), Llama-style (causal), BERT (masked LM)."""
from .bert import BertConfig, BertMLM, mask_tokens
from .gpt2 import GPT2, GPT2Config
from .llama import Llama, LlamaConfig

REGISTRY = {
    "gpt2-small": (GPT2, GPT2Config),
    "gpt2-tiny": (GPT2, GPT2Config.tiny),
    "llama-1.2b": (Llama, LlamaConfig),
    "llama-tiny": (Llama, LlamaConfig.tiny),
    "bert-base": (BertMLM, BertConfig),
    "bert-large": (BertMLM, BertConfig.large),
    "bert-tiny": (BertMLM, BertConfig.tiny),
}


def build_model(name: str):
    cls, cfg = REGISTRY[name]
    return cls(cfg())
