// Stand-in for the reference's src/lib/config.h, which pulls in the whole (absent) saiga library.  PointBlending.h
// needs nothing from it beyond the HD macro that compat/saiga/core/math/Types.h already defines.
#pragma once
