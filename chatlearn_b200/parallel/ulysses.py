"""Ulysses sequence parallelism: the sequence split is traded for a head split
around attention with two all-to-alls.

Parity: chatlearn/models/patches/transformers/qwen3_patch.py:27-106 and
chatlearn/utils/communication_op.py:69-122.  The reference patches HF attention
and issues three a2a (q, k, v) before RoPE and one after attention; KV heads are
replicated when ``sp > n_kv``.  Here the same exchange is two methods on a
group object the attention block calls.
"""

from .groups import Group


class UlyssesGroup:
    def __init__(self, group: Group):
        self.group = group
        self.size, self.rank = group.size, group.rank

    def seq_to_heads(self, x, kv: bool = False):
        """``[T_local, n, d]`` (all heads, my tokens) → ``[T_full, n/sp, d]``."""
        sp = self.size
        Tl, n, d = x.shape
        if n % sp != 0:
            assert kv and sp % n == 0, f"{n} heads cannot be split over sp={sp}"
            x = x.repeat_interleave(sp // n, dim=1)
            n = sp
        x = x.reshape(Tl, sp, n // sp, d).permute(1, 0, 2, 3).contiguous()
        y = self.group.all_to_all(x.view(sp * Tl, n // sp, d))
        return y

    def heads_to_seq(self, x):
        """``[T_full, n/sp, d]`` → ``[T_local, n, d]``."""
        sp = self.size
        Tf, nl, d = x.shape
        Tl = Tf // sp
        y = self.group.all_to_all(x.contiguous())
        return y.view(sp, Tl, nl, d).permute(1, 0, 2, 3).reshape(Tl, sp * nl, d)

    def split(self, x, dim=0):
        """This rank's contiguous slice of a full-length tensor."""
        n = x.shape[dim] // self.size
        return x.narrow(dim, self.rank * n, n)

    def gather(self, x, dim=0):
        return self.group.gather_seq(x, dim)
