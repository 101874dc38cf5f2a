"""Algorithm interface (chatlearn/algorithm/base_algo.py): validate + run."""
from abc import ABC, abstractmethod


class BaseAlgorithm(ABC):
    @abstractmethod
    def run(self):
        ...

    def validate(self):
        pass
