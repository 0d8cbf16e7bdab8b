
"(ãêsDU®ÄŒtÍEÚ'DWQeÄYôĞÄQôÄ3vÂNKBÄñ³ÄBPlus214_Output_0