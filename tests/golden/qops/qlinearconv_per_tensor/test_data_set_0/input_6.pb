"
×#=By_scale