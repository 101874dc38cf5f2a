#!/bin/bash
# llama2-7b-rlhf: run from the repository root.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=llama2-7b-rlhf
launch rlhf --config-file template/rlhf_fsdp.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/rlhf_prompts/train.jsonl \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Llama-2-7b-hf/ \
    models.reward.load=${CHATLEARN}/pretrained_models/Llama-2-7b-rm/ \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
