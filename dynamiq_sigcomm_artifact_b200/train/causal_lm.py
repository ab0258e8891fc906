"""Causal-LM training entry point (GPT-2 small, the 1.2 B Llama-style model).

Counterpart of testbed_evaluation/train_llm_causal.py (and of the accuracy loop in
simulations_llm/distributed_llm_clm.py), on synthetic token ids and random-init weights:

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m dynamiq_sigcomm_artifact_b200.train.causal_lm --model_name llama-1.2b \
        --aggregation_method dynamiQ_aee_5bit --per_device_train_batch_size 4 --block_size 2048
"""
from .run import main as _main


def main(argv=None):
    return _main("causal", argv, default_model="gpt2-small", default_seq=1024, default_batch=8)


if __name__ == "__main__":
    main()
