"""``from models.imf_dit_video import IMFDiTVideo`` as in the reference."""
