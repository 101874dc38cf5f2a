#!/bin/bash
# qwen3-next-grpo: gated delta-net hybrid (Qwen3-Next-80B-A3B); run from the repository root.
# The rollout engine keeps a fixed-size recurrent state per sequence for the linear-attention
# layers; experts are spread over the 8 rollout ranks.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen3-next-grpo
launch grpo --config-file template/grpo_fsdp.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    runtime_args.num_episode=200 \
    runtime_args.sample_per_episode=2048 \
    runtime_args.train_global_batch_size=2048 \
    runtime_args.train_micro_batch_size=64 \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen3-Next-80B-A3B-Instruct/ \
    models.policy_trainer.packing=True \
    models.policy_trainer.max_token_in_packing=8192 \
    models.policy_trainer.groupgemm=True \
    models.policy_trainer.ulysses_sequence_parallel_size=1 \
    models.policy_trainer.save_hf=False \
    models.policy_trainer.optimizer.lr=2e-6 \
    models.policy.expert_model_parallel_size=8 \
    models.policy.max_prompt_tokens_length=1024 \
    models.policy.max_response_tokens_length=8192 \
    models.policy.num_inference_per_prompt=32 \
    models.policy.gpu_memory_utilization=0.85 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
