"""Stand-in for the absent ``argcomplete`` package (shell completion is optional)."""


def autocomplete(parser, *args, **kwargs):
    return None
