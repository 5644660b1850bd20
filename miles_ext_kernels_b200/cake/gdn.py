"""Chunked gated delta rule (GDN), forward and backward, K = V = 128, packed sequences and context parallelism, on
hand-written sm_100a kernels.

:func:`chunk_gated_delta_rule` has the signature and autograd contract of FLA's ``chunk_gated_delta_rule`` (v0.5.2),
as the reference's entry point does (reference: miles_ext_kernels/cake/gdn.py:33-65,
miles_ext_kernels/cake/_impl/gdn/ops.py:2420-2501).  A call runs, by its ``cp_context``:

- no ``cp_context``: the single-GPU kernels (forward: prep, WY transform, state scan, output; backward: adjoint scan
  and the fused gradient tail);
- a :class:`KcpContext` (:func:`build_kcp_context`; layouts ``contiguous``, ``zigzag``, ``zigzag_per_document`` or an
  explicit fragment table): this rank's fragments of the packed batch, with the chunk state crossing the cuts -- rank
  to rank, or as affine fragment summaries that one all-gather shares (:func:`kcp_chunk_gated_delta_rule` calls it
  directly).

:func:`packed_qkv_views` splits one packed row ``[.., (2 H + HV) * 128]`` into q, k, v views that the op reads in place
and whose gradients come back as one packed row (no copies on either side; not among the reference's exports of
this module: its context-parallel packages offer it).

Under any ``cp_context`` the contract is FLA's: no initial state, no final state, and the context's boundaries.

Both variants (``det``, ``fast``) run the same kernels here: every reduction has a fixed order and no kernel uses a
value atomic, so identical inputs give identical bits on the same GPU model and build.  ``--cake-gdn-recompute-state``
recomputes the WY and state tapes in the backward instead of keeping them.  ``--cake-gdn-scan-segments`` overrides the
scan planner, which cuts long sequences into segments scanned in parallel when a call has fewer (sequence, value
head) chains than the GPU has SMs.

Importing this module imports neither torch nor the kernels.
"""

from ._runtime.spec import Flag, OpSpec, lazy_exports

OP = OpSpec(
    name="gdn",
    summary="chunked gated delta rule, forward + backward, K = V = 128, packed sequences, context parallelism",
    variants=("det", "fast"),
    selected_by=(("linear_attention_backend", "cake"),),
    packages=("libmek_b200",),
    exports=("KcpContext", "build_kcp_context", "chunk_gated_delta_rule", "kcp_chunk_gated_delta_rule",
             "packed_qkv_views"),
    flags=(
        Flag(
            "--cake-gdn-recompute-state",
            dict(
                action="store_true",
                default=False,
                help=(
                    "Recompute w/u/h/v_new in the backward instead of keeping them on the autograd tape: less "
                    "activation memory, more backward time. The gradients are the bits of the saved backward."
                ),
            ),
        ),
        Flag(
            "--cake-gdn-kcp-exchange",
            dict(
                choices=("auto", "sequential", "parallel"),
                default="auto",
                help=(
                    "How the chunk state crosses rank boundaries under context parallelism: 'sequential' hands it "
                    "from rank to rank (the single-rank bits on chunk-aligned boundaries; rank r waits for rank "
                    "r - 1), 'parallel' has every rank summarise its boundary fragment as an affine map, shares the "
                    "summaries with one all-gather and folds them locally (ranks work at once), 'auto' takes "
                    "'parallel' from three ranks on."
                ),
            ),
        ),
        Flag(
            "--cake-gdn-scan-segments",
            dict(
                type=int,
                default=0,
                help=(
                    "Segments per long sequence in the two state scans: 0 lets the scan planner decide from the "
                    "layout, the head count and the SM count (it cuts sequences when there are fewer chains than "
                    "SMs), 1 forces the serial scans, N > 1 forces N segments."
                ),
            ),
        ),
    ),
)

__all__, __getattr__, __dir__ = lazy_exports(__name__, OP)
