"""Training executor: turns the episode buffer into optimizer steps.

Parity: chatlearn/runtime/trainer.py:57-105.  Step ``i`` on data-parallel rank
``r`` trains on mini-batch ``r * num_iteration + i`` of the stream dataset (the
episode is sliced by DP rank first, then into iterations).
"""

from chatlearn_b200.runtime.executor import Executor


from chatlearn_b200.utils.trace import span  # noqa: E402

class Trainer(Executor):
    def __init__(self, model_flow):
        super().__init__(model_flow)
        self.iteration = 0
        self._data_loader = None
        self._metric_prefix = "trainer"
        self.num_training_epoch = 1

    def set_data_loader(self, data_loader):
        self._data_loader = data_loader

    def setup(self):
        super().setup()
        self.num_training_epoch = int(self.global_args.runtime_args.num_training_epoch)

    def num_iteration(self) -> int:
        return self._data_loader.num_iteration()

    def set_start_iteration(self, it: int):
        self.iteration = it

    def train(self, episode: int):
        loader = self._data_loader
        trainable = [n.model for n in self.model_flow.model_nodes]
        dp_sizes = {m.data_parallel_size for m in trainable}
        assert len(dp_sizes) == 1, "models trained in one flow must share the data-parallel size"
        loader.set_dp_size(dp_sizes.pop())
        n_iter = self.num_iteration()
        for epoch in range(self.num_training_epoch):
            if epoch > 0:
                loader.shuffle()
            for it in range(n_iter):
                for node in self.model_flow.linear_order():
                    m = node.model
                    if not m.is_member:
                        continue
                    batch = loader.minibatch(m.data_parallel_rank, it)
                    first = epoch == 0 and it == 0
                    last = epoch == self.num_training_epoch - 1 and it == n_iter - 1
                    fg = m.module_args.free_gpu_memory
                    frees = m.is_colocate and (fg.offload_weights or fg.free_grad_buffers
                                               or fg.offload_optimizer_states)
                    if first and frees:
                        with span(f"train.{m.name}.onload"):
                            m.onload()
                        if m.device.type == "cuda":
                            import torch
                            m._logger.debug(f"train onload: {torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated")
                    m.timers("train_step").start()
                    with span(f"train.{m.name}.train_step"):
                        m.train_step(batch, iteration=self.iteration)
                    m.timers("train_step").stop()
                    if last and frees:
                        with span(f"train.{m.name}.offload"):
                            m.offload()
                self.iteration += 1
