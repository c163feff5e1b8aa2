"""Driver for the reference's own Blackwell kernel built by oracle/build_ref.py (test infrastructure only).

It fills the reference's flat ABI -- ``struct MoEABI``, 49 x int64, ``candidate/nvfp4_moe.cu:6598-6616`` -- the way
the reference's Python host does for its default large-batch chain (``candidate/solution.py:1496-1562``): route
count R = T*K > 1536 selects GEMM1 rung 97 and GEMM2 rung 81 (both 128-row tiles), the routed rows are pre-gathered
(``hidq_g`` / ``hidsf_g``), split-K is off. The workspace sizes follow ``candidate/solution.py:918-1003``. Only this
chain is driven; smaller batches use other rungs of the reference and are not covered here.
Used by the GPU parity test (second opinion next to the CPU oracle) and by the benchmark's comparison line.
"""
import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libnvfp4_moe_ref.so")

ABI_FIELDS = ("ids scores hid_q hid_sf w1_q w1_sf w2_q w2_sf alpha beta limit out counts fill offs toffs ptok pslot pexp "
              "route_of texp tm0 hid_bf fc1 act rout T K E H I Rmax max_tiles act_type has_limit bm cfg stream cfg2 part sk "
              "hidq_g hidsf_g cnt cnt_n acc32 small_thresh zflag zflag_host").split()
assert len(ABI_FIELDS) == 49


def available() -> bool:
    return os.path.exists(LIB)


class ReferenceKernel:
    def __init__(self):
        if not available():
            raise RuntimeError("oracle/_ref/libnvfp4_moe_ref.so is missing (build it with oracle/build_ref.py)")
        # the reference captures a CUDA graph on its second identical call; keep the eager chain for A/B clarity
        os.environ.setdefault("NVFP4_MOE_NO_GRAPH", "1")
        self.lib = C.CDLL(LIB)
        self.lib.moe_init.argtypes = [C.c_int64]
        self.lib.moe_run.argtypes = [C.c_void_p]
        self._init_done = False
        self._ws = {}

    def run(self, ids, scores, hid_q, hid_sf, w1_q, w1_sf, w2_q, w2_sf, alpha, beta, limit, out, activation_type=3):
        """All arguments are CUDA tensors in the operator's storage formats; writes ``out`` (bf16 [T, H]) asynchronously."""
        t, k = ids.shape
        e, two_i, half_h = w1_q.shape
        h, i = half_h * 2, two_i // 2
        r = t * k
        if r <= 1536 or e > 256 or h % 256 or i % 256:
            raise ValueError("this driver covers the reference's large-batch chain only (T*K > 1536, E <= 256, H, I % 256 == 0)")
        stream = torch.cuda.current_stream().cuda_stream
        if not self._init_done:
            code = self.lib.moe_init(stream)
            if code:
                raise RuntimeError(f"moe_init failed with CUDA error {code}")
            self._init_done = True
        tiles = (r + 127) // 128 + min(e, r)
        key = (t, k, e, h, i)
        ws = self._ws.get(key)
        if ws is None:
            dev, i32 = ids.device, torch.int32
            ws = dict(counts_fill=torch.zeros(2 * e, dtype=i32, device=dev), offs=torch.empty(e + 1, dtype=i32, device=dev),
                      toffs=torch.empty(e + 1, dtype=i32, device=dev), ptok=torch.empty(r, dtype=i32, device=dev),
                      pslot=torch.empty(r, dtype=i32, device=dev), pexp=torch.empty(r, dtype=i32, device=dev),
                      route_of=torch.empty(r, dtype=i32, device=dev), texp=torch.empty(tiles, dtype=i32, device=dev),
                      tm0=torch.empty(tiles, dtype=i32, device=dev), act=torch.empty(r * i, dtype=torch.bfloat16, device=dev),
                      rout=torch.empty(r * h, dtype=torch.bfloat16, device=dev),
                      gath=torch.empty(r * h * 9 // 16, dtype=torch.uint8, device=dev))
            self._ws[key] = ws
        p = lambda x: 0 if x is None else x.data_ptr()
        v = dict.fromkeys(ABI_FIELDS, 0)
        v.update(ids=p(ids), scores=p(scores), hid_q=p(hid_q), hid_sf=p(hid_sf), w1_q=p(w1_q), w1_sf=p(w1_sf), w2_q=p(w2_q),
                 w2_sf=p(w2_sf), alpha=p(alpha), beta=p(beta), limit=p(limit), out=p(out), counts=ws["counts_fill"].data_ptr(),
                 fill=ws["counts_fill"].data_ptr() + 4 * e, offs=p(ws["offs"]), toffs=p(ws["toffs"]), ptok=p(ws["ptok"]),
                 pslot=p(ws["pslot"]), pexp=p(ws["pexp"]), route_of=p(ws["route_of"]), texp=p(ws["texp"]), tm0=p(ws["tm0"]),
                 act=p(ws["act"]), rout=p(ws["rout"]), T=t, K=k, E=e, H=h, I=i, Rmax=r, max_tiles=tiles,
                 act_type=int(activation_type), has_limit=0 if limit is None else 1, bm=128, cfg=97, stream=stream, cfg2=81, sk=1,
                 hidq_g=ws["gath"].data_ptr(), hidsf_g=ws["gath"].data_ptr() + r * h // 2, small_thresh=3000)
        abi = (C.c_int64 * 49)(*[int(v[name]) for name in ABI_FIELDS])
        code = self.lib.moe_run(C.addressof(abi))
        if code:
            raise RuntimeError(f"moe_run (reference kernel) failed with code {code}")
        return out
