"""Evaluation executor (chatlearn/runtime/evaluator.py:74-132): runs the eval flow
over the whole evaluation set and hands the results to ``post_process``."""

from chatlearn_b200.runtime.executor import Executor


class Evaluator(Executor):
    def __init__(self, model_flow):
        super().__init__(model_flow)
        self._dataset = None
        self._post_process_func = None
        self._metric_prefix = "eval"
        self.is_eval = True

    def set_dataset(self, dataset):
        self._dataset = dataset
        return self

    def set_post_process_func(self, fn):
        self._post_process_func = fn
        return self

    def setup(self):
        super().setup()
        m = self.first_model()
        if m.is_member and self._dataset is not None:
            total = sum(len(d) for d in self._dataset)
            m._build_dataloader(self._dataset, total, is_eval=True)

    def eval(self, episode_id: int = None, train_iteration: int = None, return_last: bool = True):
        m = self.first_model()
        if m.is_member:
            m.reset_eval_data_iter()
        res = self.execute_flow(lambda model: model.next_batch(is_eval=True), episode_id or 0,
                                is_eval=True)
        results = {n.name: [lst] for n, lst in res.items()}
        eval_info = {"episode_iteration": episode_id, "train_iteration": train_iteration}
        if self._post_process_func is not None:
            results = self._post_process_func(results, eval_info)
        else:
            results = self.post_process(results, eval_info)
        return results

    def post_process(self, results, eval_info):
        return results
