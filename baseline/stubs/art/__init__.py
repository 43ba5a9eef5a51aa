"""Stand-in for `art` (ASCII banners), which this image lacks."""


def text2art(text, *args, **kwargs):
    return str(text)
