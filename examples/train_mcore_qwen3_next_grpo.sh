#!/bin/bash
# qwen3-next-mcore-grpo: gated delta-net hybrid under the Megatron-style trainer (tensor, pipeline and expert parallel:
# the heads of the delta-net and gated-attention layers are split over the tensor-parallel ranks); run on every node
# from the repository root (NNODES x 8 GPUs, at least 4 nodes for PP=4 x EP=8).
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen3-next-mcore-grpo
launch grpo --config-file template/grpo_megatron.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    models.policy_trainer.num_gpu=$((num_device * ${NNODES:-4})) \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen3-Next-80B-A3B-Instruct/ \
    models.policy_trainer.tensor_model_parallel_size=4 \
    models.policy_trainer.pipeline_model_parallel_size=4 \
    models.policy_trainer.expert_model_parallel_size=8 \
    models.policy_trainer.expert_tensor_parallel_size=1 \
    models.policy.expert_model_parallel_size=8 \
    models.policy.max_response_tokens_length=8192 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
