"""Show image files side by side in a notebook (parity: reference
``src/art/utils/old_benchmarking/display_image_grid.py:3-10``)."""
from __future__ import annotations

from html import escape


def image_grid_html(image_paths: list[str], images_per_row: int = 2) -> str:
    cells = "".join(f"<img src='{escape(p, quote=True)}' style='max-width: 100%; height: auto;'>" for p in image_paths)
    return (f"<div style='display: grid; grid-template-columns: repeat({int(images_per_row)}, 1fr); gap: 10px;'>"
            f"{cells}</div>")


def display_image_grid(image_paths: list[str], images_per_row: int = 2) -> str:
    """Displays the grid when IPython is available; always returns the HTML."""
    html = image_grid_html(image_paths, images_per_row)
    try:
        from IPython.display import HTML, display

        display(HTML(html))
    except ImportError:
        pass
    return html
