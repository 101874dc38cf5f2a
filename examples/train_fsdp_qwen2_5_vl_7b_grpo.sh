#!/bin/bash
# qwen2.5-vl-7b-grpo (Geometry3K): run from the repository root.
# Dataset: python -m chatlearn_b200.data.data_preprocess.geo3k --input_dir dataset/geometry3k --local_dir dataset/geo3k
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen2_5-vl-7b-grpo
launch grpo --config-file template/grpo_fsdp.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.model_type=vlm \
    runtime_args.data_path=${CHATLEARN}/dataset/geo3k/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/geo3k/test.json \
    runtime_args.sample_per_episode=1024 \
    runtime_args.train_global_batch_size=1024 \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen2.5-VL-7B-Instruct/ \
    models.policy_trainer.ulysses_sequence_parallel_size=1 \
    models.policy.max_prompt_tokens_length=2048 \
    models.policy.max_response_tokens_length=2048 \
    models.policy_trainer.train_vision_tower=True \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
