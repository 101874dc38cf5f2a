"""Free-port hand-out (chatlearn/schedule/port_manager.py:20-39), process-local."""
import threading

from chatlearn_b200.utils.utils import get_free_port


class PortManager:
    def __init__(self, port_list=None):
        self._ports = list(port_list or [])
        self._idx = 0
        self._lock = threading.Lock()
        self._given = set()

    def get_free_port(self, address="127.0.0.1") -> int:
        with self._lock:
            while self._idx < len(self._ports):
                p = self._ports[self._idx]
                self._idx += 1
                if p not in self._given:
                    self._given.add(p)
                    return p
            for _ in range(64):
                p = get_free_port(address)
                if p not in self._given:
                    self._given.add(p)
                    return p
        raise RuntimeError("no free port")
