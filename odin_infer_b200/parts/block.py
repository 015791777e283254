"""How a layer's parts are arranged."""
from __future__ import annotations

from .base import (Block, Combined, Normed, PartSpec, ResidualAdded, Scaled, Several, build_part, register_part, split_update,
                   update_factor)


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x -> x + Mixer(Norm(x)) -> x + FeedForward(Norm(x)) (infer/forward.odin:51, :117-139), then the
    block's extras in order (each sees the residual stream with everything before it added).

    Each residual add is carried out by the norm that follows it: the block hands
    the update it has not yet added to whoever runs next.  A block may have no feed-forward
    (and then no second norm).

    post_norm_mixer / post_norm_feed_forward: a plain RMSNorm on the sublayer's output before it is added,
    x -> x + Norm_b(Mixer(Norm(x))); the update travels as `Normed` to the norm that runs next, whose kernel sums the
    sublayer's terms, norms them, adds and norms again.  No product then adds itself to x in its epilogue."""

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec | None, norm_mixer: PartSpec,
                 norm_feed_forward: PartSpec | None, extras: tuple = (), post_norm_mixer: PartSpec | None = None,
                 post_norm_feed_forward: PartSpec | None = None):
        if (feed_forward is None) != (norm_feed_forward is None):
            raise ValueError("a block has a feed-forward and its norm, or neither")
        self.post_mixer = build_part("norm", post_norm_mixer) if post_norm_mixer is not None else None
        self.post_ffn = build_part("norm", post_norm_feed_forward) if (post_norm_feed_forward is not None
                                                                        and feed_forward is not None) else None
        for post in (self.post_mixer, self.post_ffn):
            if post is not None and (getattr(post, "groups", 1) != 1 or not hasattr(post, "weight")):
                raise TypeError("a norm on a sublayer's output is a plain RMSNorm")
        self._mixer = build_part("mixer", mixer)
        self.ffn = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.norm_mixer = build_part("norm", norm_mixer)
        self.norm_ffn = build_part("norm", norm_feed_forward) if norm_feed_forward is not None else None
        self.extras = [build_part("block_extra", e) for e in extras]

    @property
    def mixer(self):
        return self._mixer

    def _parts(self):
        return tuple(p for p in (self.norm_mixer, self._mixer, getattr(self, "post_mixer", None), self.norm_ffn, self.ffn,
                                 getattr(self, "post_ffn", None), *self.extras) if p is not None)

    def params(self):
        return [p for part in self._parts() for p in part.params()]

    def bind(self, tensors, rt):
        for part in self._parts():
            part.bind(tensors, rt)

    def kernel_groups(self):
        return set().union(*(p.kernel_groups() for p in self._parts()))

    def notes(self, rt):
        return [n for p in self._parts() for n in p.notes(rt)]

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    @staticmethod
    def _norm(norm, rt, x, pending, **more):
        delta, bias = split_update(pending)
        if isinstance(delta, (Normed, Combined)):
            if not norm.takes_terms:
                raise TypeError(f"{type(norm).__name__} follows an update of several terms or with a norm of its own, and takes none")
        factor = update_factor(pending)
        if factor != 1.0:
            if not norm.takes_scale:
                raise TypeError(f"{type(norm).__name__} follows a block whose update carries a factor, and takes none")
            more["scale"] = factor
        if bias is None:
            return norm.forward(rt, x, delta, **more)
        if not norm.takes_bias:
            raise TypeError(f"{type(norm).__name__} follows a part whose update carries a bias, and takes none")
        return norm.forward(rt, x, delta, bias=bias, **more)

    def forward(self, rt, step, x, pending, entry):
        mixer, ffn = self._mixer, self.ffn
        h = self._norm(self.norm_mixer, rt, x, pending)
        if self.post_mixer is not None:
            pending = Normed(mixer.forward(rt, step, h, entry), self.post_mixer.weight, self.post_mixer.eps)
        else:
            pending = mixer.forward(rt, step, h, entry, residual=x) if mixer.takes_residual else mixer.forward(rt, step, h, entry)
        if ffn is not None:
            h = self._norm(self.norm_ffn, rt, x, pending)
            if self.post_ffn is not None:
                pending = Normed(ffn.forward(rt, step, h), self.post_ffn.weight, self.post_ffn.eps)
            else:
                pending = ffn.forward(rt, step, h, residual=x) if ffn.takes_residual else ffn.forward(rt, step, h)
        for extra in self.extras:
            x, pending = extra.forward(rt, step, x, pending)
        if isinstance(pending, Scaled):
            return x, pending
        delta, bias = split_update(pending)
        return x, (pending if bias is not None else delta)


@register_part("block", "parallel")
class ParallelBlock(PreNormBlock):
    """h = Norm(x);  x -> x + Mixer(h) + FeedForward(h): one norm, and both sublayers read its output.
    A block may have no feed-forward.

    norm_feed_forward: a second norm of the same x for the feed-forward, x -> x + Mixer(Norm1(x)) + FeedForward(Norm2(x)).
    residual_mult m: x -> x + m * (Mixer(..) + FeedForward(..)); the factor travels with the pending updates (`Scaled`)
    to the norm that adds them, and no product adds itself to x in its epilogue.

    Both updates stay pending (`Several`) and are added, in the order mixer, feed-forward, by the norm
    that runs next; a sublayer whose last product has added itself to x in its epilogue leaves nothing."""

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec | None, norm: PartSpec,
                 norm_feed_forward: PartSpec | None = None, residual_mult: float = 1.0):
        self._mixer = build_part("mixer", mixer)
        self.ffn = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.norm_mixer = build_part("norm", norm)
        self.norm_ffn = build_part("norm", norm_feed_forward) if (norm_feed_forward is not None and self.ffn is not None) else None
        self.extras = []
        self.residual_mult = float(residual_mult)
        if not self.norm_mixer.takes_several:
            raise TypeError(f"{type(self.norm_mixer).__name__} cannot add several pending updates")

    def forward(self, rt, step, x, pending, entry):
        mixer, ffn = self._mixer, self.ffn
        plain = self.residual_mult == 1.0   # else nothing may add itself to x unscaled
        # a second norm reads the same x, with everything before this block added: one kernel writes both where the
        # two differ in their weights alone, else the second runs after the first has updated x
        if self.norm_ffn is None:
            h = h2 = self._norm(self.norm_mixer, rt, x, pending)
        elif getattr(self.norm_mixer, "pairs_with", lambda o: False)(self.norm_ffn):
            h, h2 = self._norm(self.norm_mixer, rt, x, pending, second=self.norm_ffn)
        else:
            h = self._norm(self.norm_mixer, rt, x, pending)
            h2 = self.norm_ffn.forward(rt, x, None)
        # h is computed: a product that adds to x in its epilogue no longer changes what the sublayers read
        out = [mixer.forward(rt, step, h, entry, residual=x) if (mixer.takes_residual and plain) else mixer.forward(rt, step, h, entry)]
        if ffn is not None:
            out.append(ffn.forward(rt, step, h2, residual=x) if (ffn.takes_residual and plain) else ffn.forward(rt, step, h2))
        pending = Several()
        for upd in out:
            if isinstance(upd, Several):
                pending.extend(upd)
            elif not isinstance(upd, ResidualAdded):
                pending.append(upd)
        if not pending:
            return x, None
        return x, (pending if plain else Scaled(pending, self.residual_mult))
