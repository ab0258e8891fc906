"""Synthetic data and sampling helpers.

Stand-ins, on random token ids, for the reference's data side: fixed sampler orders
(testbed_evaluation/gen_rand.py; ``PrecomputedSampler`` in train_llm_mmlu.py:84-108), the MMLU
prompt layout (testbed_evaluation/dataset_llm_factories.py) and the accuracy metric over the four
answer letters (simulations_llm/distributed_llm_mmlu.py:341-402).
"""
from __future__ import annotations

from typing import Iterator, List, Sequence

import torch

CHOICES = ("A", "B", "C", "D")


def gen_orders(n: int, epochs: int, seed: int) -> List[List[int]]:
    """One fixed permutation of range(n) per epoch, identical on every rank."""
    g = torch.Generator().manual_seed(seed)
    return [torch.randperm(n, generator=g).tolist() for _ in range(epochs)]


class PrecomputedSampler(torch.utils.data.Sampler):
    """Yields a precomputed index order; each rank takes every `world`-th index from `rank` on."""

    def __init__(self, order: Sequence[int], rank: int = 0, world: int = 1):
        self.order = list(order)[rank::world]

    def __iter__(self) -> Iterator[int]:
        return iter(self.order)

    def __len__(self) -> int:
        return len(self.order)


def format_mmlu_prompt(question: str, choices: Sequence[str], answer: int | None = None) -> str:
    """``question`` / ``A. ...`` ... ``D. ...`` / ``Answer:`` (+ the letter when training)."""
    lines = [question.strip()] + [f"{CHOICES[i]}. {c}" for i, c in enumerate(choices)] + ["Answer:"]
    text = "\n".join(lines)
    return text + (f" {CHOICES[answer]}" if answer is not None else "")


class SyntheticMMLU(torch.utils.data.Dataset):
    """Random "prompts" whose last position must predict one of four answer tokens.

    The answer is a deterministic function of the prompt (its first token modulo 4), so a model
    can learn it and accuracy is a meaningful metric; ``answer_tokens`` are the ids standing for
    the letters A-D."""

    def __init__(self, vocab: int, seq_len: int, n: int, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.answer_tokens = torch.tensor([vocab - 4, vocab - 3, vocab - 2, vocab - 1])
        self.ids = torch.randint(0, vocab - 4, (n, seq_len), generator=g)
        self.answers = self.ids[:, 0] % 4
        self.ids[:, -1] = self.answer_tokens[self.answers]

    def __len__(self) -> int:
        return self.ids.shape[0]

    def __getitem__(self, i: int):
        labels = torch.full_like(self.ids[i], -100)
        labels[-1] = self.ids[i, -1]  # the loss is taken at the answer position only
        return self.ids[i], labels, self.answers[i]


def mmlu_accuracy(logits_before_answer: torch.Tensor, answer_tokens: torch.Tensor, answers: torch.Tensor) -> float:
    """Share of items whose highest-scoring answer letter is the right one; logits are those of
    the position that predicts the answer token, [N, vocab]."""
    pick = logits_before_answer[:, answer_tokens.to(logits_before_answer.device)].argmax(dim=1)
    return float((pick.cpu() == answers.cpu()).float().mean())
