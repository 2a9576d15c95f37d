"""One step's ragged batch as the kernels see it.

A step runs a list of entries, each a live sequence with its next tokens: a portion of a
prompt (any length from one token up) or one decoded token. All tokens of all entries are
laid out as one flat batch; per sequence the kernels get where its tokens start in the
batch, how many keys it has once this step's tokens are stored, its state slot and its
block table per layer group. Everything is int32 and lives in ONE pinned host buffer that
goes to the device in one copy.

Layout of the buffer for capacities (tokens Tc, sequences Sc, pages per sequence Pc,
logit rows Rc, groups G):

    token_ids[Tc] positions[Tc] seq_of_token[Tc] token_from[Tc] q_start[Sc+1] kv_len[Sc]
    slots[Sc] logit_rows[Rc] tables[G][Sc][Pc]

Unused token rows carry sequence -1 (kernels skip them), unused sequences have q_len 0.
`token_from[t]` is -1, or the row of the previous step's sampled tokens that token t is to
be taken from on the device (the host did not know it yet when the batch was built).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..cache.manager import Sequence


@dataclass
class StepEntry:
    """`tokens` are the next tokens of `seq` (positions seq.num_computed ...); `want` lists
    the indices among them whose logits are asked for; `hashes` are the chain hashes of the
    sequence's full pages, if its pages are to become shareable. `late` = (index among
    `tokens`, row of the previous step's samples) names a token whose id is still on the
    device: the step was put together before the step in front had been read back."""

    seq: Sequence
    tokens: list[int]
    want: list[int]
    hashes: list[int] | None = None
    late: tuple[int, int] | None = None


@dataclass
class StepBatch:
    num_tokens: int
    num_seqs: int
    max_q_len: int
    max_kv_len: int
    num_logit_rows: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    token_from: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    tables: list[torch.Tensor]
    decode_only: bool = False
    attention_splits: int | None = None   # fixed split of the keys, when a graph needs one
    late_tokens: bool = False             # whether any token id still has to come from the device


class BatchBuffers:
    """The pinned host buffer, its device twin, and the code that fills them."""

    def __init__(self, device, max_tokens: int, max_seqs: int, max_pages: int, num_groups: int,
                 pin: bool, append_only: list[bool] | None = None):
        """`append_only[g]` says that a block table of group g only ever grows at its end
        (no window gives pages back), so a row that the same sequence filled in the last
        step of the same layout needs only its new pages written."""
        self.device = torch.device(device)
        self.append_only = list(append_only) if append_only is not None else [False] * num_groups
        self._last_layout: tuple | None = None
        self._row_owner: list[list] = []
        self._row_written: list[list[int]] = []
        self._arange = np.arange(max(max_tokens, max_seqs) + 1, dtype=np.int32)
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.max_pages = max_pages
        self.num_groups = num_groups
        size = self._layout(max_tokens, max_seqs, max_pages, max_tokens)["size"]
        self.host = torch.zeros(size, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(size, dtype=torch.int32, device=self.device)
        self._copied = torch.cuda.Event() if self.device.type == "cuda" else None
        self._in_flight = False

    def _layout(self, tc: int, sc: int, pc: int, rc: int) -> dict:
        names = [("token_ids", tc), ("positions", tc), ("seq_of_token", tc), ("token_from", tc),
                 ("q_start", sc + 1),
                 ("kv_len", sc), ("slots", sc), ("logit_rows", rc),
                 ("tables", self.num_groups * sc * pc)]
        out, offset = {}, 0
        for name, count in names:
            out[name] = (offset, count)
            offset += count
        out["size"] = offset
        return out

    def build(self, entries: list[StepEntry], page_size: int, token_capacity: int | None = None,
              seq_capacity: int | None = None, page_capacity: int | None = None,
              row_capacity: int | None = None) -> StepBatch:
        """Fill the host buffer for `entries`, copy it, and return device views. The
        capacities (default: exactly what the entries need) fix the layout, so that a
        captured graph can be replayed on batches of different content. With
        `row_capacity` the entries' own `want` is set aside and logits are asked for at
        the first `row_capacity` rows of the batch."""
        num_seqs = len(entries)
        num_tokens = sum(len(e.tokens) for e in entries)
        rows = 0 if row_capacity is not None else sum(len(e.want) for e in entries)
        pages = max((len(t) for e in entries for t in e.seq.tables), default=1)
        tc = num_tokens if token_capacity is None else token_capacity
        sc = num_seqs if seq_capacity is None else seq_capacity
        pc = max(1, pages) if page_capacity is None else page_capacity
        rc = max(1, rows) if row_capacity is None else row_capacity
        if rows > rc:
            raise ValueError("more logit rows are wanted than the capacity given")
        if tc > self.max_tokens or sc > self.max_seqs or pc > self.max_pages:
            raise ValueError(
                f"step of {tc} tokens, {sc} sequences, {pc} pages per sequence exceeds the "
                f"runner's limits ({self.max_tokens}, {self.max_seqs}, {self.max_pages})"
            )
        if num_tokens > tc or num_seqs > sc or pages > pc:
            raise ValueError("the entries do not fit the capacities given")
        lay = self._layout(tc, sc, pc, rc)
        buf = self.host_np
        if self._in_flight:
            # the last step's copy reads this buffer; do not overwrite it before it ran
            self._copied.synchronize()
            self._in_flight = False

        def view(name):
            start, count = lay[name]
            return buf[start:start + count]

        token_ids, positions, seq_of = view("token_ids"), view("positions"), view("seq_of_token")
        token_from = view("token_from")
        token_from[:] = -1
        late_tokens = False
        q_start, kv_len, slots = view("q_start"), view("kv_len"), view("slots")
        logit_rows = view("logit_rows")
        tables = view("tables").reshape(self.num_groups, sc, pc)
        seq_of[:] = -1
        token_ids[num_tokens:] = 0
        positions[num_tokens:] = 0
        logit_rows[:] = 0
        if self._last_layout != (tc, sc, pc, rc):
            # another layout wrote over this region: every row starts from nothing
            self._last_layout = (tc, sc, pc, rc)
            tables[:] = -1
            self._row_owner = [[None] * sc for _ in range(self.num_groups)]
            self._row_written = [[0] * sc for _ in range(self.num_groups)]
        decode_only = all(len(e.tokens) == 1 for e in entries)
        cursor = row = 0
        max_q = max_kv = 0
        if decode_only and num_seqs:
            starts = [e.seq.num_computed for e in entries]
            count = self._arange[:num_seqs]
            token_ids[:num_seqs] = [e.tokens[0] for e in entries]
            positions[:num_seqs] = starts
            seq_of[:num_seqs] = count
            q_start[:num_seqs] = count
            kv_len[:num_seqs] = positions[:num_seqs] + 1
            slots[:num_seqs] = [e.seq.slot for e in entries]
            cursor, max_q, max_kv = num_seqs, 1, max(starts) + 1
        for index, e in enumerate(entries):
            for group, table in enumerate(e.seq.tables):
                held = len(table)
                if self._row_owner[group][index] is e.seq and self.append_only[group]:
                    written = self._row_written[group][index]
                    if held > written:
                        tables[group, index, written:held] = table[written:]
                else:
                    if self._row_owner[group][index] is not None:
                        tables[group, index, :] = -1
                    tables[group, index, :held] = table
                    self._row_owner[group][index] = e.seq
                self._row_written[group][index] = held
            n = len(e.tokens)
            base = index if decode_only else cursor
            if e.late is not None:
                token_from[base + e.late[0]] = e.late[1]
                late_tokens = True
            for w in (e.want if row_capacity is None else ()):
                if not 0 <= w < n:
                    raise ValueError(f"{e.seq.seq_id}: wanted place {w} is outside its {n} tokens")
                logit_rows[row] = base + w
                row += 1
            if decode_only:
                continue
            start = e.seq.num_computed
            token_ids[cursor:cursor + n] = e.tokens
            positions[cursor:cursor + n] = self._arange[:n] + start
            seq_of[cursor:cursor + n] = index
            q_start[index] = cursor
            kv_len[index] = start + n
            slots[index] = e.seq.slot
            cursor += n
            max_q = max(max_q, n)
            max_kv = max(max_kv, start + n)
        for group in range(self.num_groups):
            owners = self._row_owner[group]
            for index in range(num_seqs, sc):
                if owners[index] is not None:
                    tables[group, index, :] = -1
                    owners[index] = None
        if row_capacity is not None:
            rows = rc
            logit_rows[:rc] = self._arange[:rc]
        q_start[num_seqs:sc + 1] = cursor
        kv_len[num_seqs:] = 0
        slots[num_seqs:] = 0
        size = lay["size"]
        self.dev[:size].copy_(self.host[:size], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
            self._in_flight = True

        def dview(name):
            start, count = lay[name]
            return self.dev[start:start + count]

        return StepBatch(
            num_tokens=tc, num_seqs=sc, max_q_len=max_q, max_kv_len=max_kv, num_logit_rows=rows,
            token_ids=dview("token_ids"), positions=dview("positions"),
            seq_of_token=dview("seq_of_token"), token_from=dview("token_from"),
            q_start=dview("q_start"), kv_len=dview("kv_len"),
            slots=dview("slots"),
            logit_rows=dview("logit_rows")[:rows if row_capacity is None else rc],
            tables=[t for t in dview("tables").view(self.num_groups, sc, pc)],
            decode_only=decode_only, late_tokens=late_tokens,
        )
