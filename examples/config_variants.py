"""Writes the smaller example configurations, each a variation of the tiny Llama run that shows one feature
(capability parity: reference examples/{config_qwen.py, config_nanoset.yaml, config_resume_training.py, config_tiny_llama_with_s3_upload.yaml}):

    config_qwen.yaml                        a small dense Qwen2 (GQA, no MoE), dp2 x tp2 x pp2
    config_nanoset.yaml                     two data stages reading pre-tokenised files (tools/preprocess_data.py writes them), with blend weights
    config_resume_training.yaml             continues the tiny Llama run from its latest checkpoint (same layout or another one)
    config_tiny_llama_with_s3_upload.yaml   checkpoints are pushed to S3 by s5cmd after every save and removed locally

    python examples/config_variants.py
"""
import copy
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from config_tiny_llama import config as tiny  # noqa: E402

from nanotron_b200.config import DataArgs, DatasetStageArgs, NanosetDatasetsArgs, Qwen2Config, S3UploadArgs, TokenizerArgs  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def qwen():
    cfg = copy.deepcopy(tiny)
    cfg.general.run = "tiny_qwen_%date_%jobid"
    cfg.model.model_config = Qwen2Config(
        bos_token_id=1, eos_token_id=2, hidden_act="silu", hidden_size=64, intermediate_size=256, max_position_embeddings=256, num_attention_heads=8,
        num_hidden_layers=4, num_key_value_heads=4, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False, vocab_size=1024, attention_bias=True,
    )
    return cfg


def nanoset():
    cfg = copy.deepcopy(tiny)
    cfg.general.run = "tiny_llama_nanoset"
    cfg.tokenizer = TokenizerArgs(tokenizer_name_or_path="gpt2")
    cfg.model.model_config.vocab_size = 50257
    cfg.data_stages = [
        DatasetStageArgs(name="Stable Training Stage", start_training_step=1,
                         data=DataArgs(dataset=NanosetDatasetsArgs(dataset_folder="datasets/c4-es/tokenized"), seed=42, num_loading_workers=1)),
        DatasetStageArgs(name="Annealing Phase", start_training_step=10,
                         data=DataArgs(dataset=NanosetDatasetsArgs(dataset_folder=["datasets/c4-es/tokenized", "datasets/yelp/tokenized"], dataset_weights=[0.8, 0.2]), seed=42, num_loading_workers=1)),
    ]
    return cfg


def resume():
    cfg = copy.deepcopy(tiny)
    cfg.general.run = "tiny_llama_resumed"
    cfg.checkpoints.resume_checkpoint_path = "./checkpoints"  # the folder that holds latest.txt; a step folder works too
    cfg.tokens.train_steps = 30  # the schedule continues where the checkpoint stopped
    return cfg


def s3_upload():
    cfg = copy.deepcopy(tiny)
    cfg.general.run = "tiny_llama_s3"
    cfg.s3_upload = S3UploadArgs(upload_s3_path="s3://my-bucket/nanotron/tiny_llama", remove_after_upload=True, s5cmd_numworkers=16, s5cmd_concurrency=5, s5cmd_path=None)
    return cfg


VARIANTS = {"config_qwen.yaml": qwen, "config_nanoset.yaml": nanoset, "config_resume_training.yaml": resume, "config_tiny_llama_with_s3_upload.yaml": s3_upload}

if __name__ == "__main__":
    for name, build in VARIANTS.items():
        path = os.path.join(HERE, name)
        build().save_as_yaml(path)
        print(f"wrote {path}")
