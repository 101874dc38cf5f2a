#!/bin/bash
# Common environment of the example launch scripts: one process per GPU on one node.
export num_device=${num_device:-$(nvidia-smi -L 2>/dev/null | wc -l)}
[ "${num_device}" -ge 1 ] || export num_device=1
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
export OMP_NUM_THREADS=${OMP_NUM_THREADS:-8}
export TOKENIZERS_PARALLELISM=false
# symmetric memory is used with plain peer loads/stores only: keep it off NVLink multicast objects
export TORCH_SYMM_MEM_DISABLE_MULTICAST=${TORCH_SYMM_MEM_DISABLE_MULTICAST:-1}
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
# build the sm_100a extension once, in-tree
python -c "import __graft_entry__ as g; g.build()" || exit 1
launch() {   # launch <algorithm> <args...>
  if [ "${NNODES:-1}" -gt 1 ]; then
    # one launcher per node (NODE_RANK, NNODES, MASTER_ADDR, MASTER_PORT from the job environment): the launchers
    # watch each other, so a failure on any node stops the whole job
    python -m chatlearn_b200.launcher.dlc_utils --nproc-per-node "${num_device}" -- python -m chatlearn_b200 "$@"
  else
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "${num_device}" \
      --master-addr "${MASTER_ADDR}" --master-port "${MASTER_PORT}" -m chatlearn_b200 "$@"
  fi
}
