"""A stand-in for the engine, for tests of the generation loop and of the sessions
on a machine without a GPU.

The loop and the sessions are the library's (engine/generate.cpp).  They are written
against an interface (Driver) whose second implementation, beside the real engine,
is a callback: the library asks it to take and free slots, to run a pass and to
choose tokens, as JSON (api/call.cpp: "llm.open_foreign").  ``StandIn`` answers those
questions in Python; a test subclasses it to say what the "model" computes and to
check what it was asked.
"""
import ctypes
import json
import traceback

from janas_b200 import lib
from janas_b200.cache import SlotPool


class StandIn:
    vocab = 50

    def __init__(self, max_positions=40, max_tokens=64 * 4, max_seqs=3, extend=True, ahead=False):
        self.max_positions = max_positions
        self.max_tokens = max_tokens
        self.pool = SlotPool(max_seqs)
        self.extend, self.ahead = extend, ahead
        self.len = {}
        self.seeds = {}
        self.error = None
        self._reply = None
        self._cb = lib.PART_CALLBACK(self._serve)
        r = lib.call("llm.open_foreign", fn=ctypes.cast(self._cb, ctypes.c_void_p).value, user=0,
                     max_batch=max_seqs)
        self._h = ctypes.c_void_p(r["llm"])

    def close(self):
        if self._h is not None:
            lib.lib().jb_llm_close(self._h)
            self._h = None

    # ---- the protocol
    def _serve(self, user, method, args_json):
        try:
            out = getattr(self, "do_" + method.decode())(json.loads(args_json.decode()))
        except lib.CacheFull as e:
            out = {"error": str(e), "code": lib.EFULL}
        except AssertionError as e:
            traceback.print_exc()
            self.error = e
            out = {"error": f"the stand-in's check failed: {e}"}
        except Exception as e:
            traceback.print_exc()
            out = {"error": f"{type(e).__name__}: {e}"}
        self._reply = ctypes.create_string_buffer(json.dumps(out or {}).encode())
        return ctypes.cast(self._reply, ctypes.c_void_p).value

    def do_vocab_size(self, a): return {"value": self.vocab}
    def do_max_positions(self, a): return {"value": self.max_positions}
    def do_free_slots(self, a): return {"value": self.pool.n_free}
    def do_free_tokens(self, a): return {"value": self.max_tokens}
    def do_supports_extend(self, a): return {"ok": self.extend}
    def do_decodes_ahead(self, a): return {"ok": self.ahead}

    def do_new_sequence(self, a):
        s = self.pool.take()
        self.len[s] = 0
        self.on_new(s)
        return {"slot": s}

    def do_free_sequence(self, a):
        try:
            self.pool.give_back(a["slot"])
        except RuntimeError as e:
            if "no pool" in str(e):     # the interpreter is ending: the pool went first
                return {}
            raise
        del self.len[a["slot"]]
        self.on_free(a["slot"])
        return {}

    def do_length(self, a): return {"value": self.len[a["slot"]]}

    def do_truncate(self, a): return {"ok": self.truncate(a["slot"], a["n"])}

    def do_set_samplers(self, a):
        for s, o in zip(a["slots"], a["settings"]):
            self.seeds[s] = o["seed"]
        return {}

    def do_run(self, a):
        return {"tokens": self.run(a["entries"]), "forced": 0}

    # ---- for subclasses
    def on_new(self, slot): pass
    def on_free(self, slot): pass

    def truncate(self, slot, n):
        self.len[slot] = n
        return True

    def run(self, entries):
        raise NotImplementedError
