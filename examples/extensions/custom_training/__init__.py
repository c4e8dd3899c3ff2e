"""An extension package: components a service loads at start, under the package's own ids.

    SHADOWSPILL_EXTENSIONS=examples.extensions.custom_training python -m shadowspill_b200.server --root runs/

A service imports every module named in ``SHADOWSPILL_EXTENSIONS`` (comma separated) and calls its
``register(registry)``. Components are versioned (``name@version``); an id that is already taken is
refused, so an extension cannot silently replace a built-in. Clients then name the new components
like any other: ``Model("acme/llama3-wide@1")``, ``Preparation(policies=[Policy("acme/short_rows@1")])``.
The component listing (``ServiceClient.list_components``) shows each with the distribution that
provided it and a digest of its source.

Workers receive resolved settings (an explicit architecture, plain numbers), not component ids, so
they need nothing from this package.
"""
from dataclasses import replace


def register(registry) -> None:
    from shadowspill_b200.models.config import preset

    def wide():
        """The tiny Llama with twice the feed-forward width: a new architecture under a new name."""
        base = preset("llama3-tiny")
        return replace(base, d_ff=2 * base.d_ff)

    registry.add_model("acme/llama3-wide@1", wide, capabilities=("text", "packed"))
    # a policy preset: row chunks of 128 tokens and the output projection in four blocks
    registry.add_policy("acme/short_rows@1",
                        lambda rows=128, projection=4: {"alias_of": "shadowspill/text_chunks@1",
                                                        "projection": projection, "moe": 0, "rows": rows,
                                                        "delta_heads": 1})
