"""Entry point with the reference's script name: ``python prepare_wan_syn.py convert ...``."""
from imfvideo_b200.data.prepare_wan_syn import *  # noqa: F401,F403
from imfvideo_b200.data.prepare_wan_syn import main

if __name__ == "__main__":
    main()
