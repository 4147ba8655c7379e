#pragma once
namespace boost { namespace serialization { class access; }}
