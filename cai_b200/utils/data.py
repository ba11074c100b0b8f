"""Token-file batches for the device trainer.

A corpus is one flat file of token ids (``uint16`` or ``uint32``, raw or ``.npy``), memory-mapped. The batch of optimizer
step ``s`` is a pure function of ``(seed, s)``: ``rows`` windows of ``seq + 1`` tokens whose start offsets come from a
counter-based generator keyed by the seed and the step; tokens are the first ``seq`` ids of a window, targets the last
``seq`` (next-token prediction). Consequences: every data-parallel rank computes the same global list and keeps its own
rows, nothing has to be communicated; resuming from a checkpoint needs no loader state beyond the step number; two runs
with the same seed see the same data whatever their parallel layout.

A background thread prepares the next steps into (pinned, when a GPU is present) host buffers while the current step
runs, so the file reads never sit between two steps. The reference has no data path at all (its trainers draw synthetic
tokens: tools/gpu_trainer.c, tools/reftrain.c); ``synthetic_batch`` remains the default here too.
"""
from __future__ import annotations

import queue
import threading
from pathlib import Path

import numpy as np
import torch


def open_tokens(path, dtype=None) -> np.ndarray:
    """Memory-map a token file. ``.npy`` files carry their dtype; raw files are ``uint16`` unless ``dtype`` says otherwise."""
    path = Path(path)
    if path.suffix == ".npy":
        arr = np.load(path, mmap_mode="r")
        if arr.ndim != 1:
            arr = arr.reshape(-1)
    else:
        arr = np.memmap(path, dtype=np.dtype(dtype or "uint16"), mode="r")
    if arr.dtype.kind not in "ui":
        raise ValueError(f"{path}: token ids must be integers, found {arr.dtype}")
    return arr


class TokenBatches:
    """Deterministic next-token batches out of a token file, one data-parallel rank's rows at a time."""

    def __init__(self, path, vocab: int, seq: int, rows_global: int, seed: int, dp: int = 1, dp_id: int = 0, dtype=None,
                 prefetch: int = 2, pin: bool | None = None):
        if rows_global % dp:
            raise ValueError("the global batch must divide over the data-parallel ranks")
        self.tokens = open_tokens(path, dtype)
        self.vocab, self.seq, self.rows_global, self.seed = int(vocab), int(seq), int(rows_global), int(seed)
        self.rows = rows_global // dp
        self.lo = dp_id * self.rows
        self.windows = len(self.tokens) - (seq + 1)
        if self.windows <= 0:
            raise ValueError(f"{path}: {len(self.tokens)} tokens are fewer than one window of {seq + 1}")
        self.pin = torch.cuda.is_available() if pin is None else pin
        # the prefetch thread pins its buffers in the CUDA context of the rank's own device, not of device 0
        self._device = torch.cuda.current_device() if (self.pin and torch.cuda.is_available()) else None
        self._q, self._next, self._thread, self._stop = None, None, None, False
        self._depth = max(0, int(prefetch))

    def offsets(self, step: int) -> np.ndarray:
        """Start offsets of the global batch of ``step`` (the same on every rank)."""
        rng = np.random.Generator(np.random.Philox(key=self.seed & 0xFFFFFFFFFFFFFFFF, counter=[0, 0, 0, int(step)]))
        return rng.integers(0, self.windows, size=self.rows_global, dtype=np.int64)

    def make(self, step: int):
        """This rank's ``(tokens, targets)`` of ``step``: int32 tensors ``[rows, seq]``."""
        offs = self.offsets(step)[self.lo:self.lo + self.rows]
        win = np.stack([np.asarray(self.tokens[o:o + self.seq + 1]) for o in offs]).astype(np.int64)
        if win.max(initial=0) >= self.vocab:
            raise ValueError(f"token id {int(win.max())} in the data is outside the model's vocabulary of {self.vocab}")
        tok = torch.from_numpy(win[:, :-1].astype(np.int32))
        tgt = torch.from_numpy(win[:, 1:].astype(np.int32))
        if self.pin:
            tok, tgt = tok.pin_memory(), tgt.pin_memory()
        return tok, tgt

    # ---- prefetching -------------------------------------------------------------------------------------------
    def _run(self, first):
        if self._device is not None:
            torch.cuda.set_device(self._device)
        step = first
        while not self._stop:
            try:
                item = (step, self.make(step), None)
            except Exception as e:  # handed to the consumer, which raises it
                item = (step, None, e)
            while not self._stop:
                try:
                    self._q.put(item, timeout=0.1)
                    break
                except queue.Full:
                    continue
            step += 1

    def get(self, step: int):
        """The batch of ``step``; consecutive calls are served from the prefetch queue, anything else restarts it."""
        if self._depth == 0:
            return self.make(step)
        if self._thread is None or self._next != step:
            self.close()
            self._stop = False
            self._q = queue.Queue(maxsize=self._depth)
            self._thread = threading.Thread(target=self._run, args=(step,), daemon=True)
            self._thread.start()
        got, batch, err = self._q.get()
        assert got == step
        self._next = step + 1
        if err is not None:
            raise err
        return batch

    def close(self):
        if self._thread is not None:
            self._stop = True
            self._thread.join(timeout=5.0)
            self._thread = None
            self._q = None
            self._next = None


def main(argv=None):
    """``python -m cai_b200.utils.data TEXT OUT.bin``: a byte-level corpus (ids 0..255, uint16) out of any file, enough to
    train on real text without a tokenizer; files tokenized elsewhere are used as they are."""
    import argparse
    ap = argparse.ArgumentParser(description="write a byte-level token file (uint16 ids 0..255) from any file")
    ap.add_argument("source")
    ap.add_argument("out")
    a = ap.parse_args(argv)
    raw = np.fromfile(a.source, dtype=np.uint8)
    raw.astype(np.uint16).tofile(a.out)
    print(f"{a.out}: {len(raw):,} tokens, vocabulary 256")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
