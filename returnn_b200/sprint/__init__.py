"""
The side of the RASR ("Sprint") bridge that runs inside the RASR process: RASR embeds a Python interpreter, imports the module
named by its ``pymod-name`` option and calls fixed entry points of it. Parity: returnn/sprint/.
"""
