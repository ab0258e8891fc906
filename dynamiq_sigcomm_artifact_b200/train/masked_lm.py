"""Masked-LM training entry point (BERT-base / BERT-large).

Counterpart of testbed_evaluation/train_llm_maskedlm_bert.py: token ids uniform in the vocabulary,
15 % of the positions masked per step (80 % [MASK], 10 % random, 10 % unchanged):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m dynamiq_sigcomm_artifact_b200.train.masked_lm --aggregation_method dynamiQ_aee_4bit_fixed_butterfly
"""
from .run import main as _main


def main(argv=None):
    return _main("mlm", argv, default_model="bert-base", default_seq=512, default_batch=16)


if __name__ == "__main__":
    main()
