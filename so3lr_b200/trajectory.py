"""Trajectory and observable output of an MD loop without stalling the device.

The reference collects, once per cycle of its MD loop, the positions, momenta and box of the state plus the requested
observables of `energy_fn(..., has_aux=True)` (so3lr/cli/so3lr_md.py:1345-1390, 1895-1898), keeps `save_buffer` cycles in
host lists and then writes them to an HDF5 store or an extended-XYZ file (so3lr/cli/so3lr_md.py:227-486, 1899-1921).  Each
collection is a blocking device-to-host copy between two cycles.

`FrameSink.append` takes the same record as device tensors and returns at once: the arrays are copied into a slot of a ring of
pinned host buffers -- a device-side snapshot on the producing stream (the integrator overwrites positions in place), then the
device-to-host copy on a copy stream -- an event marks the slot, and a writer thread waits for that event and formats the frame
while the next cycle's kernels run.  `append` only blocks when every slot of the ring is
still waiting to be written (the disk is slower than the simulation).

Formats:
  extxyz  text, one frame after the other: atom count, a comment line with Lattice / Properties / per-frame scalars, one row
          per atom (species, position, momenta, per-atom observables).  Key names follow the reference's writer: `charges`
          for partial_charges, `hirsh_ratios` for hirshfeld_ratios, other per-atom observables under their own names,
          `dipole_vec` in the comment line (so3lr/cli/so3lr_md.py:449-466).
  npy     one `<name>.npy` file per array in a directory (positions, momenta, box and every observable), grown frame by frame
          with a fixed-size header that is rewritten at close, readable with numpy.load(..., mmap_mode='r'): the role of the
          chunked HDF5 datasets of so3lr/cli/so3lr_md.py:266-307 (h5py is not a dependency of this package).
"""
from __future__ import annotations

import os
import queue
import threading
from typing import Dict, Optional, Sequence

import numpy as np
import torch

SYMBOLS = {1: "H", 2: "He", 3: "Li", 4: "Be", 5: "B", 6: "C", 7: "N", 8: "O", 9: "F", 10: "Ne", 11: "Na", 12: "Mg", 13: "Al",
           14: "Si", 15: "P", 16: "S", 17: "Cl", 18: "Ar"}
PER_ATOM_KEYS = {"partial_charges": "charges", "hirshfeld_ratios": "hirsh_ratios"}


class _NpyColumn:
    """An .npy file that grows along its first axis: the header is written with room for the final frame count."""
    HEADER = 256

    def __init__(self, path, frame_shape, dtype):
        self.path, self.frame_shape, self.dtype, self.n = path, tuple(frame_shape), np.dtype(dtype), 0
        self.f = open(path, "wb")
        self._write_header()

    def _write_header(self):
        d = "{'descr': '%s', 'fortran_order': False, 'shape': %s, }" % (self.dtype.str, str((self.n,) + self.frame_shape))
        pad = self.HEADER - 10 - len(d) - 1
        if pad < 0:
            raise ValueError("frame shape too long for the header")
        head = b"\x93NUMPY\x01\x00" + int(self.HEADER - 10).to_bytes(2, "little") + (d + " " * pad + "\n").encode("latin1")
        self.f.seek(0)
        self.f.write(head)
        self.f.seek(0, os.SEEK_END)

    def append(self, a):
        a = np.ascontiguousarray(a, dtype=self.dtype).reshape(self.frame_shape)
        self.f.write(a.tobytes())
        self.n += 1

    def close(self):
        self._write_header()
        self.f.close()


class FrameSink:
    """Asynchronous writer of MD frames.

    atomic_numbers: (n,) of the structure; path: output file (extxyz) or directory (npy); observables: names of the per-frame
    observables that `append` will receive (per-atom arrays of length n, or small per-frame vectors such as dipole_vec);
    indices: subset of atoms to write (the reference's `output_atom_indices`); slots: frames in flight between device and disk.
    """

    def __init__(self, path, atomic_numbers, fmt: str = "extxyz", observables: Sequence[str] = (), indices=None, slots: int = 4,
                 momenta: bool = True, exist_ok: bool = False):
        if fmt not in ("extxyz", "npy"):
            raise ValueError("fmt must be 'extxyz' or 'npy'")
        self.path, self.fmt, self.observables, self.with_momenta = str(path), fmt, tuple(observables), bool(momenta)
        Z = np.asarray(atomic_numbers, dtype=np.int64).reshape(-1)
        self.n = int(Z.size)
        self.idx = None if indices is None else np.asarray(indices, dtype=np.int64)
        Zs = Z if self.idx is None else Z[self.idx]
        self.symbols = [SYMBOLS.get(int(z), "X") for z in Zs]
        if os.path.exists(self.path) and not exist_ok:
            # the reference refuses to overwrite a trajectory unless told to (so3lr/cli/so3lr_md.py:259-263)
            raise RuntimeError(f"File exists: {self.path}. Set exist_ok=True to override file.")
        if fmt == "npy":
            os.makedirs(self.path, exist_ok=True)
            self._cols: Dict[str, _NpyColumn] = {}
        else:
            os.makedirs(os.path.dirname(os.path.abspath(self.path)) or ".", exist_ok=True)
            self._file = open(self.path, "w")
        self.slots = max(1, int(slots))
        self._ring = [None] * self.slots           # per slot: dict name -> (pinned host tensor, device snapshot or None)
        self._free = queue.Queue()
        for s in range(self.slots):
            self._free.put(s)
        self._todo = queue.Queue()
        self._copy_stream = None
        self._error: Optional[BaseException] = None
        self.frames_written = 0
        self._thread = threading.Thread(target=self._writer, daemon=True)
        self._thread.start()

    # ---- producer side ----
    def append(self, positions, momenta=None, box=None, observables: Optional[Dict[str, torch.Tensor]] = None, step: Optional[int] = None):
        """Queue one frame.  Tensors may live on the device (copied asynchronously, ordered after the work already enqueued on the
        current stream) or on the host.  box: None, (3,), or (3, 3) with lattice vectors as rows."""
        if getattr(self, "_closed", False):
            raise RuntimeError("the sink is closed")
        if self._error is not None:
            raise RuntimeError("trajectory writer failed") from self._error
        rec = {"positions": positions}
        if self.with_momenta and momenta is not None:
            rec["momenta"] = momenta
        for k in self.observables:
            if observables is None or k not in observables:
                raise KeyError(f"observable '{k}' was announced but not given")
            rec[k] = observables[k]
        slot = self._free.get()                    # blocks only when every slot is still waiting for the disk
        bufs = self._ring[slot] or {}
        event = None
        cuda_src = [t for t in rec.values() if torch.is_tensor(t) and t.is_cuda]
        dev = cuda_src[0].device if cuda_src else None
        if cuda_src and self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=dev)
        staged = []
        for k, t in rec.items():
            t = t if torch.is_tensor(t) else torch.as_tensor(np.asarray(t))
            t = t.detach()
            b = bufs.get(k)
            if b is None or b[0].shape != t.shape or b[0].dtype != t.dtype or (b[1] is None) == t.is_cuda:
                # pinned host buffer and, for device sources, a device snapshot buffer of the slot
                b = (torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda), torch.empty_like(t) if t.is_cuda else None)
                bufs[k] = b
            if t.is_cuda:
                # snapshot on the producing stream (the integrator updates positions in place on that stream right after this
                # call), device-to-host from the snapshot on the copy stream
                b[1].copy_(t, non_blocking=True)
                staged.append(b)
            else:
                b[0].copy_(t)
        if staged:
            self._copy_stream.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(self._copy_stream):
                for host, snap in staged:
                    host.copy_(snap, non_blocking=True)
            event = torch.cuda.Event()
            event.record(self._copy_stream)
        self._ring[slot] = bufs
        cell = None if box is None else np.asarray(box.detach().cpu() if torch.is_tensor(box) else box, dtype=np.float64)
        self._todo.put((slot, event, list(rec.keys()), cell, step))

    def close(self):
        """Write what is in flight and close the files (a second call does nothing)."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        self._todo.put(None)
        self._thread.join()
        if self.fmt == "npy":
            for c in self._cols.values():
                c.close()
        else:
            self._file.close()
        if self._error is not None:
            raise RuntimeError("trajectory writer failed") from self._error

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    # ---- writer thread ----
    def _writer(self):
        while True:
            item = self._todo.get()
            if item is None:
                return
            slot, event, keys, cell, step = item
            try:
                if self._error is None:
                    if event is not None:
                        event.synchronize()
                    frame = {k: self._ring[slot][k][0].numpy() for k in keys}
                    if self.fmt == "npy":
                        self._write_npy(frame, cell)
                    else:
                        self._write_extxyz(frame, cell, step)
                    self.frames_written += 1
            except BaseException as e:  # surfaced by the next append / close
                self._error = e
            finally:
                self._free.put(slot)

    def _select(self, a):
        return a if (self.idx is None or a.shape[:1] != (self.n,)) else a[self.idx]

    def _write_npy(self, frame, cell):
        if cell is not None:
            frame = dict(frame, box=np.asarray(cell, dtype=np.float32))
        for k, a in frame.items():
            a = self._select(np.asarray(a))
            a = a.astype(np.float32) if a.dtype.kind == "f" else a
            col = self._cols.get(k)
            if col is None:
                col = self._cols[k] = _NpyColumn(os.path.join(self.path, k + ".npy"), a.shape, a.dtype)
            col.append(a)

    def _write_extxyz(self, frame, cell, step):
        pos = self._select(np.asarray(frame["positions"], dtype=np.float64))
        cols, props = [pos], "species:S:1:pos:R:3"
        if "momenta" in frame:
            cols.append(self._select(np.asarray(frame["momenta"], dtype=np.float64)))
            props += ":momenta:R:3"
        info = []
        for k in self.observables:
            a = np.asarray(frame[k], dtype=np.float64)
            if a.shape[:1] == (self.n,) and a.size == self.n:
                cols.append(self._select(a.reshape(self.n))[:, None])
                props += f":{PER_ATOM_KEYS.get(k, k)}:R:1"
            else:
                info.append(f'{k}="' + " ".join(repr(float(v)) for v in a.reshape(-1)) + '"')
        head = []
        if cell is not None:
            c = np.diag(cell) if cell.shape == (3,) else (np.eye(3) * float(cell.reshape(-1)[0]) if cell.size == 1 else cell.reshape(3, 3))
            head.append('Lattice="' + " ".join(repr(float(v)) for v in c.reshape(-1)) + '"')
        head.append("Properties=" + props)
        head += info
        if step is not None:
            head.append(f"step={int(step)}")
        head.append('pbc="T T T"' if cell is not None else 'pbc="F F F"')
        table = np.concatenate(cols, axis=1)
        lines = [str(len(self.symbols)), " ".join(head)]
        fmt = " ".join(["%.8f"] * table.shape[1])
        lines += [s + " " + (fmt % tuple(row)) for s, row in zip(self.symbols, table)]
        self._file.write("\n".join(lines) + "\n")


def read_extxyz(path):
    """Frames of a file written by FrameSink: list of dicts with numbers of atoms, symbols, the comment-line entries and the
    per-atom columns by name.  A reader for tests and post-processing; the format is the one ase.io.read(..., format='extxyz')
    parses."""
    import re
    frames, lines, i = [], open(path).read().split("\n"), 0
    while i < len(lines) and lines[i].strip():
        n = int(lines[i])
        comment = lines[i + 1]
        info = {m.group(1): m.group(2) if m.group(2) is not None else m.group(3)
                for m in re.finditer(r'(\w+)=(?:"([^"]*)"|(\S+))', comment)}
        spec = info["Properties"].split(":")
        names, widths = spec[0::3], [int(v) for v in spec[2::3]]
        rows = [ln.split() for ln in lines[i + 2: i + 2 + n]]
        fr = {"n": n, "info": info, "symbols": [r[0] for r in rows]}
        col = 1
        for name, w in zip(names[1:], widths[1:]):
            fr[name] = np.array([[float(v) for v in r[col: col + w]] for r in rows]).reshape(n, w) if w > 1 else \
                np.array([float(r[col]) for r in rows])
            col += w
        if "Lattice" in info:
            fr["cell"] = np.array([float(v) for v in info["Lattice"].split()]).reshape(3, 3)
        frames.append(fr)
        i += 2 + n
    return frames
